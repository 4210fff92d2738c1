"""The CPU oracle against the fixtures generated from the reference
(tests/golden/make_golden.py): every code of every sub-byte type, the encode
rounding probes, dtype ranges and the 16x16 weight-tile placement."""
import json
import os

import numpy as np
import pytest

from oracle import quant_oracle as qo
from tilus_b200 import dtypes as D


@pytest.fixture(scope="module")
def kat(golden_dir):
    return np.load(os.path.join(golden_dir, "cast_kat.npz"))


@pytest.fixture(scope="module")
def meta(golden_dir):
    with open(os.path.join(golden_dir, "dtype_meta.json")) as f:
        return json.load(f)


def _golden_names(kat, prefix):
    return sorted(k.split("/", 1)[1] for k in kat.files if k.startswith(prefix + "/"))


def test_decode_every_code(kat):
    names = _golden_names(kat, "decode")
    assert len(names) == 13 + 14
    for name in names:
        dt = D.weight_dtype(name)
        np.testing.assert_array_equal(qo.decode_table(dt), kat[f"decode/{name}"], err_msg=name)


def test_decoded_values_exact_in_fp16():
    for dt in D.ALL_WEIGHT_DTYPES:
        t = qo.decode_table(dt)
        # 5-exponent-bit types: the top binade lies outside [min_value, max_value]
        # (floats_subbyte.py:41-44 of the reference) and is never produced by quantization
        t = t[np.abs(t) <= float(dt.max_value)]
        assert np.array_equal(t.astype(np.float16).astype(np.float64), t), dt.name


def test_encode_rounding_probes(kat):
    for name in _golden_names(kat, "encode"):
        dt = D.weight_dtype(name)
        got = qo.encode_float_codes(kat[f"probes/{name}"], dt)
        np.testing.assert_array_equal(got.astype(np.int64), kat[f"encode/{name}"], err_msg=name)


def test_encode_decode_round_trip():
    for dt in D.ALL_WEIGHT_DTYPES:
        if not dt.is_float() or dt.exponent_nbits == 5:
            continue
        codes = np.arange(1 << dt.nbits)
        vals = qo.decode_codes(codes, dt)
        back = qo.encode_float_codes(vals, dt)
        # -0 keeps its sign bit
        np.testing.assert_array_equal(back, codes.astype(np.uint8), err_msg=dt.name)


def test_dtype_ranges(meta):
    for name, m in meta.items():
        dt = D.weight_dtype(name)
        assert dt.nbits == m["nbits"]
        assert float(dt.min_value) == float(m["min"]), name
        # the reference's uint4b/uint3b/uint2b declare max 16/8/4 (metadata off by one);
        # the value range of the codes themselves is 2^b - 1
        if name in ("uint4b", "uint3b", "uint2b"):
            assert m["max"] == dt.max_value + 1
        else:
            assert float(dt.max_value) == float(m["max"]), name


def test_tile_layout_matches_reference_algebra(golden_dir):
    g = np.load(os.path.join(golden_dir, "tile_layout.npz"))
    lane, slot = g["lane"], g["slot"]
    for b in range(1, 9):
        fl_lane, fl_local = g[f"flat_lane/{b}"], g[f"flat_local/{b}"]
        # byte position of (lane, lane-local byte j) from the reference's flattened layout
        pos = {(int(l), int(j)): p for p, (l, j) in enumerate(zip(fl_lane, fl_local))}
        bmap = qo.ref_tile_bit_map(b)
        for k in range(16):
            for n in range(16):
                for bit in range(b):
                    lane_bit = int(slot[k, n]) * b + bit
                    want = pos[(int(lane[k, n]), lane_bit // 8)] * 8 + lane_bit % 8
                    assert bmap[k, n, bit] == want, (b, k, n, bit)


@pytest.mark.parametrize("b", range(1, 9))
def test_pack_round_trips(b):
    rng = np.random.default_rng(b)
    codes = rng.integers(0, 1 << b, size=(32, 48), dtype=np.uint8)
    st = qo.pack_canonical(codes, b)
    assert st.size == 32 * 48 * b // 8
    np.testing.assert_array_equal(qo.unpack_canonical(st, b, codes.size).reshape(codes.shape), codes)
    tiled = qo.pack_ref_tiled(codes, b)
    assert tiled.size == st.size
    np.testing.assert_array_equal(qo.unpack_ref_tiled(tiled, b, 32, 48), codes)


def test_canonical_bit_addressing_known_answer():
    # element i occupies bits [3i, 3i+3): codes 1,2,3,4,5,6,7,0 ->
    # bits: 100 010 110 001 101 011 111 000 (LSB first)
    codes = np.array([[1, 2, 3, 4, 5, 6, 7, 0]], dtype=np.uint8)
    st = qo.pack_canonical(codes, 3)
    stream = 0
    for i, c in enumerate(codes.reshape(-1)):
        stream |= int(c) << (3 * i)
    assert list(st) == [(stream >> (8 * j)) & 0xFF for j in range(3)]


def test_dequantize_single_rounding_and_zero_point():
    rng = np.random.default_rng(0)
    K, N, g = 256, 32, 128
    codes = rng.integers(0, 16, size=(K, N), dtype=np.uint8)
    scales = rng.uniform(0.005, 0.02, size=(K // g, N)).astype(np.float16)
    w = qo.dequantize(codes, scales, D.uint4b, g, zero_point=8)
    want = ((codes.astype(np.float64) - 8) * np.repeat(scales.astype(np.float64), g, axis=0)).astype(np.float16)
    np.testing.assert_array_equal(w.view(np.uint16), want.view(np.uint16))
    # uint4 with zero point 8 == int4 whose two's-complement code is q ^ 8
    w2 = qo.dequantize(codes ^ 8, scales, D.int4b, g)
    np.testing.assert_array_equal(w.view(np.uint16), w2.view(np.uint16))


def test_quantize_weight_int_and_float():
    rng = np.random.default_rng(1)
    w = rng.standard_normal((64, 256)).astype(np.float32)
    for dt in (D.int4b, D.int3b, D.float6_e3m2):
        codes, scales = qo.quantize_weight(w, dt, 128)
        assert codes.shape == (256, 64) and scales.shape == (2, 64)
        deq = qo.dequantize(codes, scales, dt, 128).astype(np.float32)
        err = np.abs(deq - w.T).max() / np.abs(w).max()
        assert err < (0.2 if dt.nbits == 3 else 0.1), (dt.name, err)
