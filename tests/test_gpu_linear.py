"""QuantizedLinear (the reference's operator surface) on the GPU, against the oracle."""
import numpy as np
import pytest
import torch

from oracle import quant_oracle as qo
from tilus_b200 import QuantizedLinear, float16
from tilus_b200 import dtypes as D
from tilus_b200 import packing

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dt", [D.int4b, D.int3b, D.int6b, D.int8, D.float6_e3m2, D.float4_e2m1, D.float3_e1m1,
                                D.float8_e5m2], ids=lambda d: d.name)
@pytest.mark.parametrize("m", [1, 16, 33])
def test_load_and_quantize_forward(dt, m):
    """Mirrors the reference example's own check (examples/quantization/matmul_a16wx.py:590-607)
    and tightens it: the kernel output must match the oracle's quantize -> dequantize -> matmul."""
    torch.manual_seed(0)
    k, n, group = 1024, 256, 128
    layer = QuantizedLinear(x_dtype=float16, w_dtype=dt, group_size=group, in_features=k, out_features=n).cuda()
    a = ((torch.rand(m, k) - 0.5) / np.sqrt(k)).to(torch.float16)
    b = ((torch.rand(k, n) - 0.5) / np.sqrt(k)).to(torch.float16)
    layer.load_and_quantize(b.T.contiguous())
    c = layer(a.cuda())
    torch.cuda.synchronize()
    assert c.shape == (m, n) and c.dtype == torch.float16 and c.is_cuda

    codes, scales = qo.quantize_weight(b.T.contiguous().numpy(), dt, group)
    np.testing.assert_array_equal(layer.codes().cpu().numpy(), codes)
    np.testing.assert_array_equal(layer.scales.data.cpu().numpy().view(np.uint16), scales.view(np.uint16))
    w = qo.dequantize(codes, scales, dt, group)
    np.testing.assert_array_equal(layer.dequantized_weight().cpu().numpy().view(np.uint16), w.view(np.uint16))
    ref = qo.gemm_fp16(a.numpy(), w).astype(np.float64)
    got = c.cpu().numpy().astype(np.float64)
    assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-2
    # the reference example's own (loose) criterion against the unquantized product
    if dt.nbits >= 6:
        torch.testing.assert_close(c.cpu(), (a.float() @ b.float()).half(), atol=1e-2, rtol=1e-2)


def test_load_packed_reference_formats():
    torch.manual_seed(1)
    k, n, group = 512, 64, 128
    dt = D.int4b
    codes = torch.randint(0, 16, (k, n), dtype=torch.int32).to(torch.uint8)
    scales = (torch.rand(k // group, n) * 0.015 + 0.005).to(torch.float16)
    a = torch.randn(4, k).to(torch.float16)
    ref = qo.quantized_matmul(a.numpy(), codes.numpy(), scales.numpy(), dt, group).astype(np.float64)
    for layout, storage in (
        ("canonical", torch.from_numpy(qo.pack_canonical(codes.numpy(), 4))),
        ("ref_tiled", torch.from_numpy(qo.pack_ref_tiled(codes.numpy(), 4))),
        ("k_major", torch.from_numpy(qo.pack_along_k(codes.numpy(), 4))),
    ):
        layer = QuantizedLinear(float16, dt, group, k, n).cuda()
        layer.load_packed(storage.cuda(), scales.cuda(), layout=layout)
        got = layer(a.cuda()).cpu().numpy().astype(np.float64)
        assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-2, layout


def test_state_dict_round_trip():
    k, n = 512, 32
    layer = QuantizedLinear(float16, D.int4b, 128, k, n).cuda()
    layer.load_and_quantize(torch.randn(n, k))
    sd = layer.state_dict()
    assert int(sd["layout_version"]) == packing.LAYOUT_VERSION
    other = QuantizedLinear(float16, D.int4b, 128, k, n).cuda()
    other.load_state_dict(sd)
    x = torch.randn(2, k, dtype=torch.float16, device="cuda")
    assert torch.equal(layer(x), other(x))


@pytest.mark.parametrize("M", [1, 5, 40, 200])
def test_forward_host_matches_forward(M):
    """Host-buffer path (b200q_gemm_host through forward_host): pinned contiguous buffers and
    strided views of pageable ones give what forward() gives on the same data."""
    k, n = 1024, 272
    layer = QuantizedLinear(float16, D.int4b, 128, k, n).cuda()
    layer.load_and_quantize(torch.randn(n, k))
    x = torch.randn(M, k).half()
    want = layer(x.cuda()).cpu().float()
    scale = float(want.abs().max())
    got = layer.forward_host(x.pin_memory())
    torch.cuda.synchronize()
    assert got.shape == (M, n) and not got.is_cuda
    assert float((got.float() - want).abs().max()) <= 2e-3 * scale
    # row-strided views (lda > K, ldc > N)
    xs = torch.zeros(M, k + 8, dtype=torch.float16)
    xs[:, :k] = x
    outs = torch.full((M, n + 16), 7.0, dtype=torch.float16)
    layer.forward_host(xs[:, :k], outs[:, :n])
    torch.cuda.synchronize()
    assert float((outs[:, :n].float() - want).abs().max()) <= 2e-3 * scale
    assert bool((outs[:, n:] == 7.0).all())
    with pytest.raises(ValueError):
        layer.forward_host(x.cuda())


@pytest.mark.parametrize("M", [1, 9])
def test_forward_host_bf16(M):
    """The host path with bfloat16 activations (the kernel's first CTAs fetch bf16 rows, the result goes to
    pinned bf16 memory)."""
    from tilus_b200 import bfloat16

    k, n = 1024, 768
    layer = QuantizedLinear(bfloat16, D.int4b, 128, k, n).cuda()
    layer.load_and_quantize(torch.randn(n, k, generator=torch.Generator().manual_seed(3)))
    x = torch.randn(M, k, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16)
    want = layer(x.cuda()).cpu().float()
    out = torch.zeros(M, n, dtype=torch.bfloat16).pin_memory()
    for _ in range(2):
        layer.forward_host(x.pin_memory(), out)
        torch.cuda.synchronize()
        assert float((out.float() - want).abs().max()) <= 1e-2 * float(want.abs().max())
        out.zero_()


def test_forward_host_decode_call_behind_a_larger_batch():
    """A decode-batch host call queued directly behind a host call for a larger batch: the second starts
    while the first still runs, so the two must not share a staging buffer (the operator layer keeps
    one per kind)."""
    k, n = 2048, 2048
    layer = QuantizedLinear(float16, D.int4b, 128, k, n).cuda()
    layer.load_and_quantize(torch.randn(n, k, generator=torch.Generator().manual_seed(8)))
    big = torch.randn(64, k, generator=torch.Generator().manual_seed(9)).half().pin_memory()
    small = torch.randn(1, k, generator=torch.Generator().manual_seed(10)).half().pin_memory()
    out_big = torch.zeros(64, n, dtype=torch.float16).pin_memory()
    out_small = torch.zeros(1, n, dtype=torch.float16).pin_memory()
    want_big = layer(big.cuda()).cpu().float()
    want_small = layer(small.cuda()).cpu().float()
    for _ in range(5):
        layer.forward_host(big, out_big)
        layer.forward_host(small, out_small)
        layer.forward_host(small, out_small)
        torch.cuda.synchronize()
        assert float((out_big.float() - want_big).abs().max()) <= 2e-3 * float(want_big.abs().max())
        assert float((out_small.float() - want_small).abs().max()) <= 2e-3 * float(want_small.abs().max())
        out_big.zero_(); out_small.zero_()


def test_forward_host_replays_from_a_cuda_graph_with_fresh_inputs():
    """Host calls captured into a CUDA graph: every replay reads what the pinned activation buffer holds
    at that time (the kernel fetches it over PCIe, nothing is baked in) and writes the pinned result."""
    k, n, M = 1024, 512, 2
    layer = QuantizedLinear(float16, D.int4b, 128, k, n).cuda()
    layer.load_and_quantize(torch.randn(n, k, generator=torch.Generator().manual_seed(5)))
    x = torch.zeros(M, k, dtype=torch.float16).pin_memory()
    outs = [torch.zeros(M, n, dtype=torch.float16).pin_memory() for _ in range(3)]
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for o in outs:
            layer.forward_host(x, o)  # warm-up on the capture stream
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for o in outs:
                layer.forward_host(x, o)
        for seed in (6, 7):
            x.copy_(torch.randn(M, k, generator=torch.Generator().manual_seed(seed)).half())
            graph.replay()
            side.synchronize()
            want = layer(x.cuda()).cpu().float()
            for o in outs:
                assert float((o.float() - want).abs().max()) <= 2e-3 * float(want.abs().max())


@pytest.mark.parametrize("M", [1, 3, 16])
def test_forward_host_back_to_back_calls_keep_their_order(M):
    """Consecutive host calls overlap on the GPU (a call with pinned activations does not wait for the
    kernel before it until it writes its outputs).  Each call must still read the activations it was
    given at the time and results must land in call order: two layers, calls queued without any
    synchronisation in between, the same output buffer written twice, inputs rewritten only after a
    synchronisation."""
    k, n = 2048, 4096
    la = QuantizedLinear(float16, D.int5b, 128, k, n).cuda()
    lb = QuantizedLinear(float16, D.int4b, 128, k, n).cuda()
    la.load_and_quantize(torch.randn(n, k, generator=torch.Generator().manual_seed(1)))
    lb.load_and_quantize(torch.randn(n, k, generator=torch.Generator().manual_seed(2)))
    xs = [torch.randn(M, k, generator=torch.Generator().manual_seed(10 + i)).half().pin_memory() for i in range(4)]
    outs = [torch.zeros(M, n, dtype=torch.float16).pin_memory() for _ in range(3)]
    for _ in range(3):  # several rounds: the later ones run from warm caches and prepared calls
        la.forward_host(xs[0], outs[0])
        lb.forward_host(xs[1], outs[1])
        la.forward_host(xs[2], outs[2])
        lb.forward_host(xs[3], outs[2])  # the same buffer again: the later call's result must stay
        la.forward_host(xs[1], outs[0])  # and outs[0] ends with la(xs[1])
        torch.cuda.synchronize()
        want = {
            0: la(xs[1].cuda()).cpu().float(),
            1: lb(xs[1].cuda()).cpu().float(),
            2: lb(xs[3].cuda()).cpu().float(),
        }
        for i, w in want.items():
            assert float((outs[i].float() - w).abs().max()) <= 2e-3 * float(w.abs().max()), i
        for o in outs:
            o.zero_()
    # a long run of calls queued at once: every call's result against forward() on the same input
    many = [torch.zeros(M, n, dtype=torch.float16).pin_memory() for _ in range(32)]
    for i, o in enumerate(many):
        (la if i % 3 else lb).forward_host(xs[i % 4], o)
    torch.cuda.synchronize()
    for i, o in enumerate(many):
        w = (la if i % 3 else lb)(xs[i % 4].cuda()).cpu().float()
        assert float((o.float() - w).abs().max()) <= 2e-3 * float(w.abs().max()), i
    from tilus_b200 import ops
    assert ops.device_status(ops.get_workspace(torch.device("cuda", 0), 1 << 20)) == [0, 0, 0, 0]


@pytest.mark.parametrize("dt", [D.int4b, D.int5b, D.int2b, D.float6_e2m3, D.float5_e2m2, D.float8_e5m2, D.uint4b],
                         ids=lambda d: d.name)
@pytest.mark.parametrize("group,wdtype", [(32, torch.float32), (128, torch.float16), (512, torch.float32)])
def test_gpu_quantize_and_pack_bit_exact(dt, group, wdtype):
    """b200q_quantize (absmax scales, clamp, round / float encode, packing in one library call)
    against the oracle's load_and_quantize arithmetic and the host re-packer, bit for bit."""
    from tilus_b200 import quantize

    torch.manual_seed(3)
    k, n = 1024, 64
    w = (torch.randn(n, k) * 0.3).to(wdtype)
    w[0, :group] = 0  # an all-zero group: the scale floor 1e-6
    w[1, 5] = 1e4     # an outlier: saturation of everything else to tiny codes
    packed, scales = quantize.quantize_and_pack(w.cuda(), dt, group)
    torch.cuda.synchronize()
    codes_ref, scales_ref = qo.quantize_weight(w.float().numpy(), dt, group)
    np.testing.assert_array_equal(scales.cpu().numpy().view(np.uint16), scales_ref.view(np.uint16))
    want = packing.interleave(torch.from_numpy(codes_ref), dt)
    assert torch.equal(packed.cpu(), want)


@pytest.mark.parametrize("k,group", [(640, 64), (1152, 128), (384, 32)])
def test_load_and_quantize_general_k(k, group):
    """GPU-side load_and_quantize and forward for in_features that are multiples of 128 only and
    scale groups below 128: codes, scales and dequantized weights bit-identical to the oracle."""
    torch.manual_seed(1)
    n, m, dt = 96, 5, D.int4b
    layer = QuantizedLinear(x_dtype=float16, w_dtype=dt, group_size=group, in_features=k, out_features=n).cuda()
    a = ((torch.rand(m, k) - 0.5) / np.sqrt(k)).to(torch.float16)
    b = ((torch.rand(k, n) - 0.5) / np.sqrt(k)).to(torch.float16)
    layer.load_and_quantize(b.T.contiguous())
    codes, scales = qo.quantize_weight(b.T.contiguous().numpy(), dt, group)
    np.testing.assert_array_equal(layer.codes().cpu().numpy(), codes)
    np.testing.assert_array_equal(layer.scales.data.cpu().numpy().view(np.uint16), scales.view(np.uint16))
    w = qo.dequantize(codes, scales, dt, group)
    np.testing.assert_array_equal(layer.dequantized_weight().cpu().numpy().view(np.uint16), w.view(np.uint16))
    got = layer(a.cuda()).cpu().numpy().astype(np.float64)
    ref = qo.gemm_fp16(a.numpy(), w).astype(np.float64)
    assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-2
