"""CPU oracle for the per-token FP8 casts that follow the gate_up projection in a decoder layer.

TEST INFRASTRUCTURE ONLY (imported by tests/ and the smoke check, never by the product package).

Restates, in numpy float32 arithmetic, the two Tilus scripts
  examples/quantization/per_token_cast.py:22-97                      (PerTokenCast)
  examples/quantization/swiglu_forward_and_per_token_cast.py:28-166  (SwiGLUForwardAndPerTokenCast)
operation for operation.  Their float32 -> float8_e4m3 cast is the C++ conversion of
__nv_fp8_e4m3 (python/tilus/hidet/include/tilus/cuda/float8_e4m3.h:6, cuda_fp8.h): round to nearest
even, saturate to +-448, NaN -> 0x7f.

Parity status: UNPINNED against the reference's own run - its check compares with the un-vendored
`tile_kernels` package (absent) and the scripts need a GPU JIT.  What is pinned: the e4m3 encode
against PyTorch's independent float8_e4m3fn conversion on all in-range inputs (tests/test_cast_oracle.py).
"""
from __future__ import annotations

import numpy as np

FP8_MAX = np.float32(448.0)


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    """uint8 e4m3 (fn: no infinities, 0x7f / 0xff = NaN) -> float32."""
    c = np.asarray(codes, dtype=np.uint8).astype(np.int32)
    s = np.where(c & 0x80, -1.0, 1.0).astype(np.float32)
    e = (c >> 3) & 0xF
    m = (c & 7).astype(np.float32)
    val = np.where(e == 0, m * np.float32(2.0 ** -9), (1.0 + m / 8.0) * np.exp2((e - 7).astype(np.float32)))
    val = np.where((c & 0x7F) == 0x7F, np.nan, val)
    return (s * val).astype(np.float32)


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float32 -> uint8 e4m3 code: round to nearest even, saturate finite values to +-448, NaN -> 0x7f
    (__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3))."""
    x = np.asarray(x, dtype=np.float32)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    a = np.abs(np.nan_to_num(x, nan=0.0, posinf=1e30, neginf=-1e30)).astype(np.float64)
    out = np.zeros(x.shape, dtype=np.uint8)
    # exponent of the binade, clamped to the subnormal binade (2^-6)
    with np.errstate(divide="ignore", invalid="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.clip(e, -6, 8)
    step = np.exp2(e - 3)                      # spacing of representable values in that binade
    q = np.rint(a / step)                      # numpy rint = round half to even
    v = q * step                               # rounded magnitude (may have moved to the next binade)
    v = np.minimum(v, 448.0)                   # saturate
    # encode v exactly
    with np.errstate(divide="ignore", invalid="ignore"):
        e2 = np.floor(np.log2(np.where(v > 0, v, 1.0)))
    e2 = np.clip(e2, -6, 8)
    is_sub = v < 2.0 ** -6
    mant = np.where(is_sub, np.rint(v / 2.0 ** -9), np.rint((v / np.exp2(e2) - 1.0) * 8.0))
    expc = np.where(is_sub, 0, e2 + 7)
    out = (expc.astype(np.int32) << 3 | mant.astype(np.int32)).astype(np.uint8)
    out = np.where(np.isnan(x), np.uint8(0x7F), out | sign)
    return out.astype(np.uint8)


def _group_scales(value: np.ndarray, group: int):
    """value float32 [T, H] -> (scale [T, H/g], inv_scale [T, H/g]) per per_token_cast.py:83-88:
    scale = absmax / 448 if absmax > 0 else 1, inv_scale = 448 / absmax if absmax > 0 else 1 (fp32 divisions)."""
    T, H = value.shape
    g = value.reshape(T, H // group, group)
    absmax = np.abs(g).max(axis=2).astype(np.float32)
    pos = absmax > 0
    safe = np.where(pos, absmax, np.float32(1.0))
    scale = np.where(pos, (safe / FP8_MAX).astype(np.float32), np.float32(1.0)).astype(np.float32)
    inv = np.where(pos, (FP8_MAX / safe).astype(np.float32), np.float32(1.0)).astype(np.float32)
    return scale, inv


def per_token_cast(x: np.ndarray, group: int = 128):
    """x [T, H] (fp16 or float32 holding the activation values) -> (e4m3 codes uint8 [T, H], scale float32
    [T, H/group]); examples/quantization/per_token_cast.py:75-97."""
    v = np.asarray(x).astype(np.float32)
    T, H = v.shape
    assert H % group == 0
    scale, inv = _group_scales(v, group)
    scaled = (v.reshape(T, H // group, group) * inv[:, :, None]).astype(np.float32)
    return e4m3_encode(scaled).reshape(T, H), scale


def swiglu_forward_and_per_token_cast(x: np.ndarray, pos_to_token_topk=None, topk_weights=None, pos_to_expert=None,
                                      clamp_value=None, group: int = 128):
    """x [T, 2H] -> (codes uint8 [T, H], scale float32 [T, H/group], valid bool [T]);
    examples/quantization/swiglu_forward_and_per_token_cast.py:110-166.

    value = silu(l) * r with l = x[:, :H], r = x[:, H:] in fp32, silu(l) = l / (exp(-l) + 1); with a clamp
    value c: l = min(l, c), r = clip(r, -c, c) (:124-132); with routing weights: rows whose
    pos_to_token_topk entry p is >= 0 are multiplied by topk_weights[p] (:137-141); rows whose
    pos_to_expert entry is negative are skipped - nothing is written for them (:108)."""
    v = np.asarray(x).astype(np.float32)
    T, H2 = v.shape
    H = H2 // 2
    l, r = v[:, :H].copy(), v[:, H:].copy()
    if clamp_value is not None:
        c = np.float32(clamp_value)
        l = np.where(l > c, c, l)
        r = np.where(r > c, c, r)
        r = np.where(r < -c, -c, r)
    silu = (l / (np.exp(-l).astype(np.float32) + np.float32(1.0))).astype(np.float32)
    value = (silu * r).astype(np.float32)
    if pos_to_token_topk is not None and topk_weights is not None:
        p = np.asarray(pos_to_token_topk).astype(np.int64)
        w = np.asarray(topk_weights, dtype=np.float32).reshape(-1)
        wrow = np.where(p >= 0, w[np.clip(p, 0, w.size - 1)], np.float32(1.0)).astype(np.float32)
        value = np.where((p >= 0)[:, None], (value * wrow[:, None]).astype(np.float32), value)
    valid = np.ones(T, dtype=bool) if pos_to_expert is None else (np.asarray(pos_to_expert) >= 0)
    scale, inv = _group_scales(value, group)
    scaled = (value.reshape(T, H // group, group) * inv[:, :, None]).astype(np.float32)
    return e4m3_encode(scaled).reshape(T, H), scale, valid
