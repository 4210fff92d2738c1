"""The per-token FP8 cast kernels (b200q_per_token_cast, b200q_swiglu_per_token_cast,
b200q_gemm_swiglu_cast) against the oracle's restatement of the reference scripts
(examples/quantization/per_token_cast.py, swiglu_forward_and_per_token_cast.py), on the shapes
those scripts benchmark.  Scales: fp32, equal to 1e-6 relative (bit-equal for the plain cast,
whose arithmetic has no transcendental).  Codes: equal, except where the device's expf and
numpy's differ in the last bit of a value that sits on a rounding boundary - at most one FP8
step, on at most one element in a thousand."""
import numpy as np
import pytest
import torch

from oracle import cast_oracle as co
from oracle import quant_oracle as qo
from tilus_b200 import QuantizedLinear, float16, ops, synth
from tilus_b200 import dtypes as D

pytestmark = pytest.mark.gpu


def _codes(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.uint8).cpu().numpy()


def _check_codes(got: np.ndarray, want: np.ndarray, exact: bool):
    if exact:
        np.testing.assert_array_equal(got, want)
        return
    diff = got != want
    assert diff.mean() <= 1e-3, diff.mean()
    if diff.any():  # neighbours in the e4m3 code order: same sign, code differs by one
        g, w = got[diff].astype(np.int32), want[diff].astype(np.int32)
        assert (np.abs(g - w) <= 1).all()


@pytest.mark.parametrize("tokens,hidden", [(128, 1024), (256, 2048), (257, 4096), (3, 512)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["f16", "bf16"])
def test_per_token_cast(tokens, hidden, dtype):
    torch.manual_seed(tokens)
    x = (torch.randn(tokens, hidden) * 2.0).to(dtype)
    x[1, :128] = 0  # an all-zero group
    out, sf = ops.per_token_cast(x.cuda(), 128)
    torch.cuda.synchronize()
    want_codes, want_sf = co.per_token_cast(x.float().numpy(), 128)
    np.testing.assert_array_equal(sf.cpu().numpy(), want_sf)
    _check_codes(_codes(out), want_codes, exact=True)


@pytest.mark.parametrize("group", [256, 512])
def test_per_token_cast_wider_groups(group):
    x = (torch.randn(17, 2048) * 3.0).to(torch.float16)
    out, sf = ops.per_token_cast(x.cuda(), group)
    want_codes, want_sf = co.per_token_cast(x.float().numpy(), group)
    np.testing.assert_array_equal(sf.cpu().numpy(), want_sf)
    _check_codes(_codes(out), want_codes, exact=True)


@pytest.mark.parametrize("tokens,hidden,num_tokens,topk", [(128, 1024, 64, 2), (256, 2048, 128, 2), (257, 4096, 128, 2),
                                                           (1024, 4096, 512, 2)])
def test_swiglu_forward_and_per_token_cast(tokens, hidden, num_tokens, topk):
    """Inputs as the reference script builds them (swiglu_forward_and_per_token_cast.py:197-246):
    x ~ 2 * N(0, 1), routing positions, uniform weights, every 17th row masked out, clamp 6."""
    torch.manual_seed(hidden)
    x = (torch.randn(tokens, hidden * 2) * 2.0).to(torch.float16)
    pos = (torch.arange(tokens, dtype=torch.int32) % (num_tokens * topk))
    w = torch.rand(num_tokens, topk, dtype=torch.float32)
    expert = torch.ones(tokens, dtype=torch.int32)
    expert[::17] = -1
    sentinel = 0x55
    xd, posd, wd, expd = x.cuda(), pos.cuda(), w.cuda(), expert.cuda()
    out, sf = ops.swiglu_forward_and_per_token_cast(xd, 128, posd, wd, expd, 6.0)
    # run again into pre-filled buffers to see that masked rows are left alone
    out.view(torch.uint8).fill_(sentinel)
    sf.fill_(-1.0)
    from tilus_b200 import _lib
    _lib.check(_lib.load().b200q_swiglu_per_token_cast(
        xd.data_ptr(), hidden * 2, out.data_ptr(), hidden, sf.data_ptr(), tokens, hidden, 128, _lib.ACT_F16,
        posd.data_ptr(), wd.data_ptr(), expd.data_ptr(), 1, 6.0, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    want_codes, want_sf, valid = co.swiglu_forward_and_per_token_cast(x.float().numpy(), pos.numpy(), w.numpy(),
                                                                      expert.numpy(), 6.0, 128)
    got_codes, got_sf = _codes(out), sf.cpu().numpy()
    np.testing.assert_allclose(got_sf[valid], want_sf[valid], rtol=1e-6, atol=0)
    _check_codes(got_codes[valid], want_codes[valid], exact=False)
    assert (got_codes[~valid] == sentinel).all() and (got_sf[~valid] == -1.0).all()
    # the reference script's own acceptance test: dequantized sums agree
    deq = lambda c, s: (co.e4m3_decode(c).reshape(c.shape[0], -1, 128) * s[:, :, None]).sum()  # noqa: E731
    np.testing.assert_allclose(deq(got_codes[valid], got_sf[valid]), deq(want_codes[valid], want_sf[valid]),
                               rtol=2e-2, atol=2.0)


def test_swiglu_without_clamp_weights_or_mask_bf16():
    x = (torch.randn(33, 1024) * 1.5).to(torch.bfloat16)
    out, sf = ops.swiglu_forward_and_per_token_cast(x.cuda(), 128)
    want_codes, want_sf, _ = co.swiglu_forward_and_per_token_cast(x.float().numpy(), group=128)
    np.testing.assert_allclose(sf.cpu().numpy(), want_sf, rtol=1e-6, atol=0)
    _check_codes(_codes(out), want_codes, exact=False)


@pytest.mark.parametrize("M", [1, 16, 200])
def test_gate_up_gemm_followed_by_swiglu_cast(M):
    """One library call: quantized gate_up projection, then SwiGLU + per-token cast of its output.  The
    cast is checked on the GEMM output the call itself produced (so that the GEMM's own tolerance does
    not enter), the GEMM output against the oracle."""
    K, H, g = 1024, 1024, 128
    prob = synth.make_problem(M, 2 * H, K, D.int4b, g, seed=M)
    layer = QuantizedLinear(float16, D.int4b, g, K, 2 * H).cuda()
    layer.load_codes(prob["codes"], prob["scales"])
    out, sf, gate_up = layer.forward_swiglu_cast(prob["a"].cuda(), 128, 6.0)
    torch.cuda.synchronize()
    ref = qo.quantized_matmul(prob["a"].numpy(), prob["codes"].numpy(), prob["scales"].numpy(), D.int4b, g, 0)
    gu = gate_up.cpu().numpy()
    assert np.abs(gu.astype(np.float64) - ref).max() / np.abs(ref).max() <= 1e-2
    want_codes, want_sf, _ = co.swiglu_forward_and_per_token_cast(gu.astype(np.float32), clamp_value=6.0, group=128)
    np.testing.assert_allclose(sf.cpu().numpy(), want_sf, rtol=1e-6, atol=0)
    _check_codes(_codes(out), want_codes, exact=False)


def test_cast_rejects_bad_shapes():
    x = torch.zeros(4, 192, dtype=torch.float16, device="cuda")
    with pytest.raises(Exception):
        ops.per_token_cast(x, 128)  # hidden not a multiple of the group
    with pytest.raises(Exception):
        ops.per_token_cast(torch.zeros(4, 1024, dtype=torch.float16, device="cuda"), 64)  # group below 128
