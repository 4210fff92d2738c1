"""bfloat16 activations (the reference operator's other a_dtype, examples/quantization/matmul_a16wx.py:35-41,
:418-419): scales, dequantized weights and outputs are bfloat16, accumulation fp32.  Dequantized
weights bit-exact with the oracle's bf16_rn(cast(q) * s); GEMM outputs within rel-err 1e-2."""
import numpy as np
import pytest
import torch

from oracle import quant_oracle as qo
from tilus_b200 import QuantizedLinear, bfloat16
from tilus_b200 import dtypes as D
from tilus_b200 import ops, packing, synth, variants

pytestmark = pytest.mark.gpu

REL_TOL = 1e-2


def _cases():
    out = []
    for dt in variants.supported_weight_dtypes():
        out.append((dt, 0))
        if dt.kind == D.KIND_UINT:
            out.append((dt, 1 << (dt.nbits - 1)))
    return out


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).cpu().numpy()


@pytest.mark.parametrize("dt,zp", _cases(), ids=lambda x: getattr(x, "name", str(x)))
@pytest.mark.parametrize("group", [32, 128])
def test_dequantize_bf16_bit_exact(dt, zp, group):
    dev = torch.device("cuda:0")
    K, N = 1024, 64
    prob = synth.make_problem(1, N, K, dt, group, seed=group + dt.nbits, symmetric_unsigned=False)
    codes = prob["codes"]
    codes.view(-1)[: 1 << dt.nbits] = torch.arange(1 << dt.nbits, dtype=torch.int32).to(torch.uint8)  # every code
    if dt.is_float() and dt.exponent_nbits == 5:
        tbl = np.abs(qo.decode_table(dt))
        bad = torch.from_numpy(~(tbl <= dt.max_value))
        codes[bad[codes.long()]] = 0
    scales = prob["scales"].to(torch.bfloat16)
    bq = packing.interleave(codes, dt).to(dev)
    w = ops.dequantize(bq, scales.to(dev), dt, group, zp)
    assert w.dtype == torch.bfloat16
    want = qo.dequantize_bf16(codes.numpy(), scales, dt, group, zp)
    np.testing.assert_array_equal(_bits(w), _bits(want))


@pytest.mark.parametrize("dt,zp", [(D.uint4b, 8), (D.int4b, 0), (D.float6_e3m2, 0), (D.int8, 0), (D.uint3b, 4)],
                         ids=lambda x: getattr(x, "name", str(x)))
@pytest.mark.parametrize("M", [1, 16, 40, 256])
def test_gemm_bf16(dt, zp, M):
    """All three kernels (M = 1 and 16: mma.sync; 40: tcgen05, weights as the 256-column operand; 256:
    tcgen05, weights in tensor memory) with bfloat16 activations, scales and outputs."""
    dev = torch.device("cuda:0")
    N, K, g = 384, 2048, 128
    prob = synth.make_problem(M, N, K, dt, g, seed=M + dt.nbits)
    a = prob["a"].to(torch.bfloat16)
    scales = prob["scales"].to(torch.bfloat16)
    bq = packing.interleave(prob["codes"], dt).to(dev)
    c = ops.quantized_matmul(a.to(dev), bq, scales.to(dev), dt, g, zp)
    torch.cuda.synchronize()
    assert c.dtype == torch.bfloat16 and tuple(c.shape) == (M, N)
    ref = qo.quantized_matmul_bf16(a, prob["codes"].numpy(), scales, dt, g, zp).double()
    got = c.cpu().double()
    assert float((got - ref).abs().max() / ref.abs().max()) <= REL_TOL


def test_bf16_large_activations_do_not_overflow_the_decode_path():
    """bfloat16 reaches magnitudes fp16 cannot hold.  The tcgen05 kernels multiply in bfloat16 and
    take them as they are; the mma.sync path (M <= 16) multiplies in fp16 and saturates
    activations at +-65504, which this pins down."""
    dev = torch.device("cuda:0")
    N, K, g, dt = 64, 512, 128, D.int4b
    prob = synth.make_problem(40, N, K, dt, g, seed=3)
    a = (prob["a"].float() * 1.0e5).to(torch.bfloat16)  # |a| up to ~4e5, beyond fp16
    scales = prob["scales"].to(torch.bfloat16)
    bq = packing.interleave(prob["codes"], dt).to(dev)
    c = ops.quantized_matmul(a.to(dev), bq, scales.to(dev), dt, g, 0)
    ref = qo.quantized_matmul_bf16(a, prob["codes"].numpy(), scales, dt, g, 0).double()
    assert float((c.cpu().double() - ref).abs().max() / ref.abs().max()) <= REL_TOL
    c1 = ops.quantized_matmul(a[:1].contiguous().to(dev), bq, scales.to(dev), dt, g, 0)
    a_sat = a[:1].float().clamp(-65504.0, 65504.0).to(torch.bfloat16)
    ref1 = qo.quantized_matmul_bf16(a_sat, prob["codes"].numpy(), scales, dt, g, 0).double()
    assert torch.isfinite(c1).all()
    assert float((c1.cpu().double() - ref1).abs().max() / ref1.abs().max()) <= REL_TOL


@pytest.mark.parametrize("dt", [D.int4b, D.float6_e3m2, D.int8], ids=lambda d: d.name)
@pytest.mark.parametrize("m", [1, 33])
def test_quantized_linear_bf16(dt, m):
    """QuantizedLinear(x_dtype=bfloat16): load_and_quantize on the GPU, scales stored as bfloat16,
    forward in bfloat16 - codes and scales bit-identical to the oracle's restatement."""
    torch.manual_seed(0)
    k, n, group = 1024, 256, 128
    layer = QuantizedLinear(x_dtype=bfloat16, w_dtype=dt, group_size=group, in_features=k, out_features=n).cuda()
    assert layer.scales.dtype == torch.bfloat16
    a = ((torch.rand(m, k) - 0.5) / np.sqrt(k)).to(torch.bfloat16)
    b = ((torch.rand(k, n) - 0.5) / np.sqrt(k)).to(torch.bfloat16)
    layer.load_and_quantize(b.T.contiguous())
    c = layer(a.cuda())
    torch.cuda.synchronize()
    assert c.shape == (m, n) and c.dtype == torch.bfloat16
    codes, scales = qo.quantize_weight(b.T.contiguous().float().numpy(), dt, group, bf16_scales=True)
    np.testing.assert_array_equal(layer.codes().cpu().numpy(), codes)
    sc_t = torch.from_numpy(scales).to(torch.bfloat16)
    np.testing.assert_array_equal(_bits(layer.scales.data), _bits(sc_t))
    w = qo.dequantize_bf16(codes, sc_t, dt, group)
    np.testing.assert_array_equal(_bits(layer.dequantized_weight()), _bits(w))
    ref = qo.gemm_bf16(a, w).double()
    assert float((c.cpu().double() - ref).abs().max() / ref.abs().max()) <= REL_TOL
