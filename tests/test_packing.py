"""Host re-packer: canonical / reference-tiled / b200 formats, checked against the
oracle's numpy restatement and against a slow, literal reading of the b200 layout."""
import numpy as np
import pytest
import torch

from oracle import quant_oracle as qo
from tilus_b200 import dtypes as D
from tilus_b200 import packing as P


@pytest.mark.parametrize("b", range(1, 9))
def test_canonical_and_ref_tiled_match_oracle(b):
    rng = np.random.default_rng(10 + b)
    codes = rng.integers(0, 1 << b, size=(32, 64), dtype=np.uint8)
    t = torch.from_numpy(codes)
    np.testing.assert_array_equal(P.pack_canonical(t, b).numpy(), qo.pack_canonical(codes, b))
    np.testing.assert_array_equal(P.pack_ref_tiled(t, b).numpy(), qo.pack_ref_tiled(codes, b))
    np.testing.assert_array_equal(
        P.unpack_canonical(torch.from_numpy(qo.pack_canonical(codes, b)), b, 32, 64).numpy(), codes
    )
    np.testing.assert_array_equal(
        P.unpack_ref_tiled(torch.from_numpy(qo.pack_ref_tiled(codes, b)), b, 32, 64).numpy(), codes
    )


def _literal_b200(codes, dt):
    """Bit-by-bit construction of the b200 layout from its written description."""
    b = dt.nbits
    K, N = codes.shape
    KB, NT = K // 512, N // 16
    out = np.zeros(K * N * b // 32, dtype=np.uint64)
    planes = P.PLANES[b]
    for nt in range(NT):
        for kb in range(KB):
            blk = (nt * KB + kb) * b * 2 * 32 * 4  # words per block
            for half in range(2):
                for r in range(8):
                    n = nt * 16 + half * 8 + r
                    for j in range(4):
                        lane = r * 4 + j
                        for c in range(4):
                            k0 = kb * 512 + c * 128 + j * 32
                            for h in range(16):
                                for e in range(2):
                                    q = int(codes[k0 + 2 * h + e, n])
                                    if dt.kind == D.KIND_INT:
                                        q ^= 1 << (b - 1)
                                    lo, base = b, 0
                                    for p in planes:
                                        lo -= p
                                        per = 16 // p
                                        v = base + h // per
                                        f = h % per
                                        field = (q >> lo) & ((1 << p) - 1)
                                        widx = blk + ((c * 2 + half) * 32 + lane) * b + v
                                        out[widx] |= np.uint64(field << (16 * e + f * p))
                                        base += p
    return out.astype(np.uint32).view(np.uint8)


@pytest.mark.parametrize("dt", [D.uint1b, D.uint2b, D.int3b, D.uint4b, D.int4b, D.uint5b, D.float6_e3m2,
                                D.int7b, D.uint8, D.int8], ids=lambda d: d.name)
def test_b200_layout_literal(dt):
    rng = np.random.default_rng(dt.nbits)
    codes = rng.integers(0, 1 << dt.nbits, size=(1024, 32), dtype=np.uint8)
    got = P.interleave(torch.from_numpy(codes), dt).numpy()
    assert got.size == codes.size * dt.nbits // 8
    np.testing.assert_array_equal(got, _literal_b200(codes, dt))
    back = P.deinterleave(torch.from_numpy(got), dt, 1024, 32).numpy()
    np.testing.assert_array_equal(back, codes)


def test_b200_column_shards_are_contiguous():
    dt = D.uint4b
    rng = np.random.default_rng(0)
    codes = rng.integers(0, 16, size=(512, 64), dtype=np.uint8)
    full = P.interleave(torch.from_numpy(codes), dt)
    for n0, n1 in ((0, 32), (32, 64), (16, 48)):
        part = P.interleave(torch.from_numpy(np.ascontiguousarray(codes[:, n0:n1])), dt)
        assert torch.equal(P.shard_columns(full, dt, 512, 64, n0, n1), part)


def test_shape_check():
    with pytest.raises(ValueError):
        P.interleave(torch.zeros(192, 16, dtype=torch.uint8), D.uint4b)  # K not a multiple of 128
    with pytest.raises(ValueError):
        P.interleave(torch.zeros(512, 24, dtype=torch.uint8), D.uint4b)


@pytest.mark.parametrize("name", ["int4b", "int3b", "float6_e3m2", "int8"])
def test_reference_checkpoint_loads_directly(name):
    """A state dict written by the reference's QuantizedLinear (quantized_weight in its
    [K/16, N/16, 32*b] tiling + scales, no layout tag) loads into this library's class; a
    checkpoint with another layout version is refused."""
    from tilus_b200 import QuantizedLinear, float16

    dt = D.weight_dtype(name)
    K, N, g = 1024, 48, 128
    gen = torch.Generator().manual_seed(5)
    codes = torch.randint(0, 1 << dt.nbits, (K, N), dtype=torch.uint8, generator=gen)
    scales = (torch.rand(K // g, N, generator=gen) * 0.015 + 0.005).half()
    ref_sd = {"quantized_weight": P.pack_ref_tiled(codes, dt.nbits), "scales": scales}
    layer = QuantizedLinear(float16, dt, g, K, N)
    layer.load_state_dict(ref_sd)
    assert torch.equal(layer.codes(), codes)
    assert torch.equal(layer.scales.data, scales)
    assert int(layer.layout_version) == P.LAYOUT_VERSION
    # own checkpoints round-trip unchanged
    other = QuantizedLinear(float16, dt, g, K, N)
    other.load_state_dict(layer.state_dict())
    assert torch.equal(other.quantized_weight.data, layer.quantized_weight.data)
    # unknown layout version: refused
    bad = dict(layer.state_dict())
    bad["layout_version"] = torch.tensor(P.LAYOUT_VERSION + 1, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="layout version"):
        QuantizedLinear(float16, dt, g, K, N).load_state_dict(bad)
