"""Weight and activation data types of the weight-only quantized matmul.

The names, bit widths and value ranges restate the reference's dtype tables
(python/tilus/hidet/ir/dtypes/integer_subbyte.py:66-98 for intNb/uintNb,
python/tilus/hidet/ir/dtypes/floats_subbyte.py:23-109 for floatN_eXmY), so a
call site written against the reference (``w_dtype=int4b``,
``w_dtype=float6_e3m2``) reads the same here.

Semantics restated:

* ``intNb``  : two's complement in N bits.
* ``uintNb`` : unsigned in N bits.
* ``floatN_eXmY`` : sign / X exponent bits / Y mantissa bits, bias 2^(X-1)-1,
  subnormals, and for X < 5 every exponent code is a finite number (no Inf/NaN).

Every value of every type with at most 8 bits is exactly representable in fp16.
"""
from __future__ import annotations

from dataclasses import dataclass

KIND_UINT = 0
KIND_INT = 1
KIND_FLOAT = 2


@dataclass(frozen=True)
class WeightDType:
    name: str
    short_name: str
    nbits: int
    kind: int
    exponent_nbits: int = 0
    mantissa_nbits: int = 0

    # --- reference-style predicates -------------------------------------
    def is_float(self) -> bool:
        return self.kind == KIND_FLOAT

    def is_integer(self) -> bool:
        return self.kind != KIND_FLOAT

    def signedness(self) -> bool:
        return self.kind != KIND_UINT

    @property
    def exponent_bias(self) -> int:
        return (1 << (self.exponent_nbits - 1)) - 1

    @property
    def min_value(self):
        if self.kind == KIND_UINT:
            return 0
        if self.kind == KIND_INT:
            return -(1 << (self.nbits - 1))
        return -self.max_value

    @property
    def max_value(self):
        if self.kind == KIND_UINT:
            return (1 << self.nbits) - 1
        if self.kind == KIND_INT:
            return (1 << (self.nbits - 1)) - 1
        e, m, bias = self.exponent_nbits, self.mantissa_nbits, self.exponent_bias
        # floats_subbyte.py:35-48: with 5 exponent bits the all-ones exponent is
        # reserved (Inf/NaN); with fewer it is an ordinary binade.
        top = (1 << e) - 1 - (1 if e == 5 else 0)
        return 2.0 ** (top - bias) * (2.0 - 2.0 ** (-m))

    @property
    def code(self) -> int:
        """Integer tag passed through the C ABI: kind<<16 | nbits<<8 | e<<4 | m."""
        return (self.kind << 16) | (self.nbits << 8) | (self.exponent_nbits << 4) | self.mantissa_nbits

    def __repr__(self) -> str:  # pragma: no cover - cosmetic
        return self.name


def _int(n: int) -> WeightDType:
    name = "int8" if n == 8 else f"int{n}b"
    return WeightDType(name, f"i{n}", n, KIND_INT)


def _uint(n: int) -> WeightDType:
    name = "uint8" if n == 8 else f"uint{n}b"
    return WeightDType(name, f"u{n}", n, KIND_UINT)


def _float(n: int, e: int, m: int) -> WeightDType:
    assert 1 + e + m == n
    return WeightDType(f"float{n}_e{e}m{m}", f"f{n}e{e}m{m}", n, KIND_FLOAT, e, m)


int1b, int2b, int3b, int4b, int5b, int6b, int7b, int8 = (_int(n) for n in range(1, 9))
uint1b, uint2b, uint3b, uint4b, uint5b, uint6b, uint7b, uint8 = (_uint(n) for n in range(1, 9))
i1, i2, i3, i4, i5, i6, i7, i8 = int1b, int2b, int3b, int4b, int5b, int6b, int7b, int8
u1, u2, u3, u4, u5, u6, u7, u8 = uint1b, uint2b, uint3b, uint4b, uint5b, uint6b, uint7b, uint8

float8_e5m2 = f8e5m2 = _float(8, 5, 2)
float7_e5m1 = f7e5m1 = _float(7, 5, 1)
float7_e4m2 = f7e4m2 = _float(7, 4, 2)
float7_e3m3 = f7e3m3 = _float(7, 3, 3)
float7_e2m4 = f7e2m4 = _float(7, 2, 4)
float6_e4m1 = f6e4m1 = _float(6, 4, 1)
float6_e3m2 = f6e3m2 = _float(6, 3, 2)
float6_e2m3 = f6e2m3 = _float(6, 2, 3)
float5_e3m1 = f5e3m1 = _float(5, 3, 1)
float5_e2m2 = f5e2m2 = _float(5, 2, 2)
float5_e1m3 = f5e1m3 = _float(5, 1, 3)
float4_e2m1 = f4e2m1 = _float(4, 2, 1)
float4_e1m2 = f4e1m2 = _float(4, 1, 2)
float3_e1m1 = f3e1m1 = _float(3, 1, 1)

ALL_WEIGHT_DTYPES = [
    int1b, int2b, int3b, int4b, int5b, int6b, int7b, int8,
    uint1b, uint2b, uint3b, uint4b, uint5b, uint6b, uint7b, uint8,
    float8_e5m2, float7_e5m1, float7_e4m2, float7_e3m3, float7_e2m4,
    float6_e4m1, float6_e3m2, float6_e2m3, float5_e3m1, float5_e2m2, float5_e1m3,
    float4_e2m1, float4_e1m2, float3_e1m1,
]
_BY_NAME = {}
for _d in ALL_WEIGHT_DTYPES:
    _BY_NAME[_d.name] = _d
    _BY_NAME[_d.short_name] = _d


@dataclass(frozen=True)
class ActDType:
    name: str
    short_name: str
    nbits: int = 16

    def __repr__(self) -> str:  # pragma: no cover - cosmetic
        return self.name


float16 = f16 = ActDType("float16", "f16")
bfloat16 = bf16 = ActDType("bfloat16", "bf16")


def weight_dtype(x) -> WeightDType:
    """Accept a WeightDType, a reference-style name ("int4b", "u4", "float6_e3m2")
    or any object exposing ``.name`` (e.g. the reference's own dtype objects)."""
    if isinstance(x, WeightDType):
        return x
    name = x if isinstance(x, str) else getattr(x, "name", None)
    if name not in _BY_NAME:
        raise ValueError(f"unsupported weight dtype: {x!r}")
    return _BY_NAME[name]


def act_dtype(x) -> ActDType:
    import torch

    if isinstance(x, ActDType):
        return x
    if x is torch.float16:
        return float16
    if x is torch.bfloat16:
        return bfloat16
    name = x if isinstance(x, str) else getattr(x, "name", None)
    for d in (float16, bfloat16):
        if name in (d.name, d.short_name):
            return d
    raise ValueError(f"unsupported activation dtype: {x!r}")


def default_zero_point(dt: WeightDType, symmetric_unsigned: bool) -> int:
    """Zero point subtracted from the decoded code before scaling.

    The reference kernel has none (matmul_a16wx.py:319-320: b = cast(q) * scale).
    Benchmarks that draw unsigned codes and dequantize as (q - 2^(b-1)) * scale
    use ``symmetric_unsigned=True``; that equals the intNb value whose
    two's-complement code is q ^ 2^(b-1).
    """
    if dt.kind == KIND_UINT and symmetric_unsigned:
        return 1 << (dt.nbits - 1)
    return 0
