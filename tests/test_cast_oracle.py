"""The cast oracle (oracle/cast_oracle.py) on the CPU: its e4m3 encode / decode against PyTorch's
independent float8_e4m3fn conversion, and the scale rule of the per-token cast."""
import numpy as np
import torch

from oracle import cast_oracle as co


def test_e4m3_decode_matches_torch_on_every_code():
    codes = np.arange(256, dtype=np.uint8)
    mine = co.e4m3_decode(codes)
    theirs = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    np.testing.assert_array_equal(np.nan_to_num(mine, nan=-999.0), np.nan_to_num(theirs, nan=-999.0))


def test_e4m3_encode_matches_torch_in_range():
    rng = np.random.default_rng(0)
    vals = co.e4m3_decode(np.arange(256, dtype=np.uint8))
    fin = np.sort(vals[np.isfinite(vals)])
    mids = ((fin[:-1].astype(np.float64) + fin[1:]) / 2).astype(np.float32)  # exact ties: round half to even
    x = np.concatenate([rng.uniform(-448, 448, 300000), rng.standard_normal(300000) * 1e-2, fin, mids,
                        np.nextafter(mids, np.float32(np.inf)), np.nextafter(mids, np.float32(-np.inf))]).astype(np.float32)
    mine = co.e4m3_encode(x)
    theirs = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    np.testing.assert_array_equal(mine, theirs)


def test_e4m3_encode_saturates_and_keeps_nan():
    got = co.e4m3_encode(np.array([500.0, -1e9, np.nan, 0.0, -0.0], dtype=np.float32))
    assert got.tolist() == [0x7E, 0xFE, 0x7F, 0x00, 0x80]


def test_per_token_cast_scale_rule():
    rng = np.random.default_rng(1)
    x = (rng.standard_normal((5, 256)) * 3).astype(np.float16)
    x[2, :128] = 0  # an all-zero group keeps scale 1
    codes, sf = co.per_token_cast(x, 128)
    assert codes.shape == (5, 256) and sf.shape == (5, 2)
    assert sf[2, 0] == 1.0 and (codes[2, :128] & 0x7F).max() == 0
    absmax = np.abs(x.astype(np.float32)).reshape(5, 2, 128).max(axis=2)
    np.testing.assert_array_equal(sf[absmax > 0], (absmax / np.float32(448.0))[absmax > 0])
    # the largest element of every non-zero group lands on +-448 exactly
    deq = np.abs(co.e4m3_decode(codes)).reshape(5, 2, 128).max(axis=2)
    assert (deq[absmax > 0] == 448.0).all()


def test_swiglu_rows_weights_and_mask():
    rng = np.random.default_rng(2)
    x = (rng.standard_normal((6, 512)) * 2).astype(np.float16)
    pos = np.array([0, 1, -1, 3, 2, 1], dtype=np.int32)
    w = rng.uniform(0.1, 1.0, size=4).astype(np.float32)
    expert = np.array([1, -1, 1, 1, 1, 1], dtype=np.int32)
    codes, sf, valid = co.swiglu_forward_and_per_token_cast(x, pos, w, expert, clamp_value=6.0, group=128)
    assert valid.tolist() == [True, False, True, True, True, True]
    plain, sf_plain, _ = co.swiglu_forward_and_per_token_cast(x, None, None, None, clamp_value=6.0, group=128)
    # a routing weight scales the group maximum, i.e. the stored scale, and leaves the codes (almost) alone
    np.testing.assert_allclose(sf[0], sf_plain[0] * w[0], rtol=1e-6)
    np.testing.assert_array_equal(sf[2], sf_plain[2])  # negative topk position: no weight
