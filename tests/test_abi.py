"""The C-ABI library loads, exports every symbol include/b200q.h declares, validates
arguments and plans shapes - all without a GPU (no compute calls here)."""
import ctypes
import os
import re

import pytest

from tilus_b200 import _lib, ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from tilus_b200 import build

    build.build()
    return _lib.load()


def test_header_symbols_are_exported_and_bound(lib):
    header = open(os.path.join(ROOT, "include", "b200q.h")).read()
    declared = set(re.findall(r"\b(b200q_[a-z_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_lib.SYMBOLS), (declared ^ set(_lib.SYMBOLS))
    for name in declared:
        assert hasattr(lib, name), name


def test_versions_and_strings(lib):
    from tilus_b200 import packing

    assert lib.b200q_version() >= 100
    assert lib.b200q_layout_version() == packing.LAYOUT_VERSION
    assert lib.b200q_status_string(0) == b"ok"
    for st in range(1, 6):
        assert lib.b200q_status_string(st)


def test_plan_static_table():
    p = ops.plan(1, 8192, 8192, "uint4b", 8, 128)
    # decode shapes run the mma.sync stream kernel: two CTAs per SM, a CTA count that divides the
    # 512 column tiles, at most half an SM's shared memory each
    assert p["kernel"] == 2 and p["splits"] * p["ctas_per_split"] <= 148 * 2
    assert (8192 // 16) % p["ctas_per_split"] == 0 and p["smem_bytes"] <= 113 * 1024 and p["stages"] >= 2
    assert p["workspace_bytes"] >= 256 + 8192 * 4
    assert ops.plan(4096, 28672, 8192, "int4b", 0, 128)["kernel"] == 1  # prefill: tcgen05 kernel
    p8 = ops.plan(8, 4096, 4096, "uint4b", 8, 128)
    assert p8["kernel"] == 2 and p8["m_tiles"] == 1 and p8["smem_bytes"] <= 113 * 1024
    # 9..16 rows: the same kernel with two 8-row activation tiles, one CTA per SM with all of its shared memory
    for m in (9, 16):
        ps = ops.plan(m, 8192, 8192, "uint4b", 8, 128)
        assert ps["kernel"] == 2 and ps["m_tiles"] == 2 and ps["smem_bytes"] <= 227 * 1024
        assert ps["splits"] * ps["ctas_per_split"] <= 148 and ps["stages"] >= 2
    # 17..128 rows: tcgen05 kernel with the weights on the 256-column side of the MMA
    for m in (17, 64, 128):
        pw = ops.plan(m, 4096, 4096, "uint4b", 8, 128)
        assert pw["kernel"] == 3 and pw["smem_bytes"] <= 227 * 1024
        assert pw["splits"] * pw["ctas_per_split"] <= 148 + 148 // 8
    assert ops.plan(129, 4096, 4096, "uint4b", 8, 128)["kernel"] == 1
    # per-channel scales, float weights
    assert ops.plan(4, 4096, 4096, "float6_e3m2", 0, 4096)["passes"] == 1


def test_rejects_bad_problems(lib):
    pl = _lib.Plan()
    u4 = (0 << 16) | (4 << 8)
    assert lib.b200q_plan(1, 8192, 8192, u4, 8, 128, ctypes.byref(pl)) == _lib.ST_OK
    assert lib.b200q_plan(1, 8192, 8192, u4, 3, 128, ctypes.byref(pl)) == _lib.ST_UNSUPPORTED  # zero point
    assert lib.b200q_plan(1, 8200, 8192, u4, 8, 128, ctypes.byref(pl)) == _lib.ST_UNSUPPORTED  # N % 16
    assert lib.b200q_plan(1, 8192, 8000, u4, 8, 128, ctypes.byref(pl)) == _lib.ST_UNSUPPORTED  # K % 512
    assert lib.b200q_plan(1, 8192, 8192, u4, 8, 48, ctypes.byref(pl)) == _lib.ST_UNSUPPORTED   # group % 32
    assert lib.b200q_plan(0, 8192, 8192, u4, 8, 128, ctypes.byref(pl)) == _lib.ST_INVALID_ARG
    assert lib.b200q_plan(1, 8192, 8192, (2 << 16) | (6 << 8) | (3 << 4) | 1, 0, 128, ctypes.byref(pl)) \
        == _lib.ST_UNSUPPORTED  # float6 with e+m != 5
    assert lib.b200q_workspace_bytes(1, 8192, 8000, u4, 8, 128) == 0
    # null pointers are refused before anything is launched
    assert lib.b200q_gemm(None, 8192, None, None, None, 8192, 1, 8192, 8192, u4, 8, 128, 0, None, 0, None) \
        == _lib.ST_INVALID_ARG
    assert lib.b200q_dequantize(None, None, None, 8192, 8192, u4, 8, 128, 0, None) == _lib.ST_INVALID_ARG
    # activation dtype tags other than fp16 (0) and bf16 (1) are refused
    assert lib.b200q_gemm(None, 8192, None, None, None, 8192, 1, 8192, 8192, u4, 8, 128, 2, None, 0, None) \
        == _lib.ST_UNSUPPORTED


def test_ops_refuse_cpu_tensors():
    import torch

    a = torch.zeros(1, 512, dtype=torch.float16)
    bq = torch.zeros(512 * 16 // 2, dtype=torch.uint8)
    sc = torch.ones(4, 16, dtype=torch.float16)
    with pytest.raises(ValueError):
        ops.quantized_matmul(a, bq, sc, "uint4b", 128, 8)
    with pytest.raises(ValueError):
        ops.dequantize(bq, sc, "uint4b", 128, 8)
