"""The kernels' bit gathering (tilus_b200/csrc/decode.cuh), compiled for the host, against
the packer: for every variant, random units must decode to code - bias (integers) or
to the oracle's float value after the fp16 arithmetic the kernels apply."""
import ctypes
import os
import subprocess
import tempfile

import numpy as np
import pytest
import torch

from oracle import quant_oracle as qo
from tilus_b200 import dtypes as D
from tilus_b200 import packing as P
from tilus_b200 import variants as V

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def harness():
    out = os.path.join(tempfile.mkdtemp(prefix="b200q_harness_"), "harness.so")
    subprocess.check_call([
        "g++", "-std=c++17", "-O1", "-shared", "-fPIC",
        "-I" + os.path.join(ROOT, "tilus_b200", "csrc"),
        os.path.join(ROOT, "tests", "decode_harness.cpp"), "-o", out,
    ])
    lib = ctypes.CDLL(out)
    lib.harness_unit_raw.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    return lib


def _cases():
    out = []
    for dt in V.supported_weight_dtypes():
        out.append((dt, 0))
        if dt.kind == D.KIND_UINT:
            out.append((dt, 1 << (dt.nbits - 1)))
    return out


@pytest.mark.parametrize("dt,zp", _cases(), ids=lambda x: getattr(x, "name", str(x)))
def test_unit_gather(harness, dt, zp):
    var = V.variant_id(dt, zp)
    assert harness.harness_var_bits(var) == dt.nbits
    assert harness.harness_var_count() == V.VARIANT_COUNT
    b = dt.nbits
    rng = np.random.default_rng(var)
    table = qo.decode_table(dt)
    for trial in range(8):
        codes = rng.integers(0, 1 << b, size=32, dtype=np.uint8)
        if trial == 0:
            codes = (np.arange(32) % (1 << b)).astype(np.uint8)
        if dt.is_float() and dt.exponent_nbits == 5:
            codes = np.where(np.abs(table[codes]) <= dt.max_value, codes, 0).astype(np.uint8)
        stored = P.stored_codes(torch.from_numpy(codes), dt)
        words = P._unit_words(stored.to(torch.int32).reshape(1, 32), b).numpy().astype(np.int32).view(np.uint32)
        words = np.ascontiguousarray(words.reshape(-1))
        raw = np.zeros(16, dtype=np.uint32)
        tgt = np.zeros(16, dtype=np.int32)
        assert harness.harness_unit_raw(var, words.ctypes.data, raw.ctypes.data, tgt.ctypes.data) == 0
        halves = np.stack([raw & 0xFFFF, raw >> 16], axis=1).astype(np.uint16).reshape(-1)  # k order
        x = halves.view(np.float16).astype(np.float64)
        t = np.repeat(tgt, 2).astype(np.float64)
        want = table[codes] - zp
        if dt.is_float():
            ebias = (1 << (dt.exponent_nbits - 1)) - 1
            got = x * 2.0 ** (15 - ebias)
        else:
            bias = harness.harness_var_bias(var)
            # stored codes are offset binary for signed types, so code - 2^(b-1) is the value
            got = x * 2.0 ** (-t) - (2.0 ** (10 - t) + bias)
            assert np.all(tgt >= 0) and np.all(tgt + b <= 10)
        np.testing.assert_array_equal(got, want)
