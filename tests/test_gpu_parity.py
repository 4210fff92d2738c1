"""GPU parity tests: the CUDA library, called through its C ABI (ctypes), against the CPU
oracle on the same seeded inputs.  Dequantized weights must match bit for bit; GEMM
outputs within rel-err 1e-2 (fp32 accumulate, fp16 out), the tolerance the task states."""
import numpy as np
import pytest
import torch

from oracle import quant_oracle as qo
from tilus_b200 import dtypes as D
from tilus_b200 import ops, packing, synth, variants

pytestmark = pytest.mark.gpu

REL_TOL = 1e-2


def _dev():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch.device("cuda:0")


def _cases():
    out = []
    for dt in variants.supported_weight_dtypes():
        out.append((dt, 0))
        if dt.kind == D.KIND_UINT:
            out.append((dt, 1 << (dt.nbits - 1)))
    return out


def _rel_err(c, ref):
    c = c.astype(np.float64)
    ref = ref.astype(np.float64)
    return np.abs(c - ref).max() / max(np.abs(ref).max(), 1e-30)


def _run(prob, M_override=None, plan_override=None):
    dev = _dev()
    dt, g, zp = prob["dtype"], prob["group_size"], prob["zero_point"]
    bq = packing.interleave(prob["codes"], dt).to(dev)
    sc = prob["scales"].to(dev)
    a = prob["a"].to(dev)
    c = ops.quantized_matmul(a, bq, sc, dt, g, zp, plan_override=plan_override)
    torch.cuda.synchronize()
    return c.cpu().numpy(), bq, sc


@pytest.mark.parametrize("dt,zp", _cases(), ids=lambda x: getattr(x, "name", str(x)))
@pytest.mark.parametrize("group", [32, 128, 1024])
def test_dequantize_bit_exact(dt, zp, group):
    dev = _dev()
    K, N = 1024, 64
    prob = synth.make_problem(1, N, K, dt, group, seed=group + dt.nbits, symmetric_unsigned=False)
    codes = prob["codes"]
    # make sure every code occurs
    codes.view(-1)[: 1 << dt.nbits] = torch.arange(1 << dt.nbits, dtype=torch.int32).to(torch.uint8)
    if dt.is_float() and dt.exponent_nbits == 5:
        tbl = np.abs(qo.decode_table(dt))
        bad = torch.from_numpy(~(tbl <= dt.max_value))
        codes[bad[codes.long()]] = 0
    bq = packing.interleave(codes, dt).to(dev)
    w = ops.dequantize(bq, prob["scales"].to(dev), dt, group, zp).cpu().numpy()
    want = qo.dequantize(codes.numpy(), prob["scales"].numpy(), dt, group, zp)
    np.testing.assert_array_equal(w.view(np.uint16), want.view(np.uint16))


@pytest.mark.parametrize("dt,zp", _cases(), ids=lambda x: getattr(x, "name", str(x)))
def test_gemm_small_all_variants(dt, zp):
    prob = synth.make_problem(5, 64, 1024, dt, 128, seed=3, symmetric_unsigned=False)
    prob["zero_point"] = zp
    c, _, _ = _run(prob)
    ref = qo.quantized_matmul(prob["a"].numpy(), prob["codes"].numpy(), prob["scales"].numpy(), dt, 128, zp)
    assert _rel_err(c, ref) <= REL_TOL


@pytest.mark.parametrize("M", [1, 2, 7, 8, 9, 16, 17, 40])
def test_gemm_ragged_m(M):
    prob = synth.make_problem(M, 128, 2048, D.uint4b, 128, seed=M)
    c, _, _ = _run(prob)
    ref = qo.quantized_matmul(prob["a"].numpy(), prob["codes"].numpy(), prob["scales"].numpy(), D.uint4b, 128, 8)
    assert c.shape == (M, 128)
    assert _rel_err(c, ref) <= REL_TOL


def _forced(M, N, K, dt, zp, override, seed=11, group=128):
    """Runs one problem twice with a forced plan on one workspace; checks parity and that the
    workspace is left zeroed."""
    dev = _dev()
    prob = synth.make_problem(M, N, K, dt, group, seed=seed)
    prob["zero_point"] = zp
    bq = packing.interleave(prob["codes"], dt).to(dev)
    # a forced plan may run another kernel than the default one for M: room for either's scratch
    need = max(ops.workspace_bytes(m, N, K, dt, zp, group) for m in (1, M, 200))
    ws = torch.zeros(need + M * N * 4, dtype=torch.uint8, device=dev)
    ref = qo.quantized_matmul(prob["a"].numpy(), prob["codes"].numpy(), prob["scales"].numpy(), dt, group, zp)
    for _ in range(2):  # second call runs on the workspace the first one left behind
        c = ops.quantized_matmul(prob["a"].to(dev), bq, prob["scales"].to(dev), dt, group, zp, workspace=ws,
                                 plan_override=override)
        torch.cuda.synchronize()
        assert _rel_err(c.cpu().numpy(), ref) <= REL_TOL
        assert int(ws.count_nonzero()) == 0, "workspace not restored to zero"


@pytest.mark.parametrize("splits,ctas", [(1, 1), (1, 5), (2, 3), (4, 8), (4, 17)])
def test_stream_kernel_shapes_and_clean_workspace(splits, ctas):
    """Kernel 2 (mma.sync, ring-fed) with forced k chunks and CTA counts: own tiles in shared
    memory, left-over tiles through the global scratch."""
    _forced(3, 272, 2048, D.int4b, 0, dict(kernel=2, splits=splits, ctas_per_split=ctas, cluster=1, stages=3, pdl=1))


@pytest.mark.parametrize("dt,zp", [(D.uint4b, 8), (D.uint3b, 4), (D.float6_e3m2, 0), (D.uint8, 0)],
                         ids=lambda x: getattr(x, "name", str(x)))
def test_stream_kernel_variants(dt, zp):
    _forced(9, 256, 1024, dt, zp, dict(kernel=2, splits=2, ctas_per_split=7, cluster=1, stages=2, pdl=1), seed=5)


@pytest.mark.parametrize("M,N,K,splits", [(9, 272, 2048, 1), (33, 272, 2048, 4), (64, 512, 1024, 2), (65, 256, 1024, 8),
                                          (128, 768, 1536, 3), (17, 16, 512, 1)])
def test_wide_kernel_shapes_and_clean_workspace(M, N, K, splits):
    """Kernel 3 (tcgen05, weights as the 256-column operand) with forced split-K factors: ragged
    last column tile (N not a multiple of 256), every activation-stage spacing (M <= 32, <= 64,
    <= 128), odd group counts per split."""
    tiles = (N + 255) // 256
    _forced(M, N, K, D.int4b, 0, dict(kernel=3, splits=splits, ctas_per_split=tiles, tile_m=128))


@pytest.mark.parametrize("dt,zp,group", [(D.uint4b, 8, 128), (D.uint3b, 4, 128), (D.float6_e3m2, 0, 1024),
                                         (D.uint8, 0, 256), (D.uint1b, 1, 128), (D.int6b, 0, 512)],
                         ids=lambda x: getattr(x, "name", str(x)))
def test_wide_kernel_variants(dt, zp, group):
    _forced(40, 528, 1024, dt, zp, dict(kernel=3, splits=2, ctas_per_split=3, tile_m=128), seed=7, group=group)


def test_wide_kernel_more_items_than_sms():
    """Persistent CTAs walk over several work items each: the pipelines, accumulator buffers and
    barrier phases carry over item boundaries."""
    M, N, K = 20, 256 * 200, 512
    prob = synth.make_problem(M, N, K, D.uint4b, 128, seed=2)
    c, _, _ = _run(prob)
    ref = qo.quantized_matmul(prob["a"].numpy(), prob["codes"].numpy(), prob["scales"].numpy(), D.uint4b, 128, 8)
    assert _rel_err(c, ref) <= REL_TOL
    assert ops.plan(M, N, K, D.uint4b, 8, 128)["kernel"] == 3


@pytest.mark.parametrize("M,N,K,splits", [(300, 256, 2048, 4), (200, 384, 1024, 2), (129, 128, 4096, 8),
                                          (520, 256, 1024, 1)])
def test_umma_kernel_forced_split_k_and_clean_workspace(M, N, K, splits):
    """Kernel 1 (tcgen05, weights in tensor memory) with forced split-K factors: several row tiles,
    a ragged last row tile, fp32 partial sums and arrival counters left zeroed."""
    m_tiles, n_tiles = (M + 255) // 256, (N + 127) // 128
    _forced(M, N, K, D.int4b, 0, dict(kernel=1, splits=splits, tile_m=256, m_tiles=m_tiles,
                                      ctas_per_split=m_tiles * n_tiles), seed=13)


@pytest.mark.parametrize("small_ws", [False, True])
def test_umma_kernel_last_round_split_along_k(small_ws):
    """160 tiles on 148 persistent CTAs: the 12 tiles of the last round are cut into K ranges whose
    partial sums meet in the fp32 scratch (left zeroed).  With a workspace too small for that scratch
    the kernel takes whole tiles instead; both must agree with the oracle."""
    dev = _dev()
    M, N, K, dt = 512, 10240, 2048, D.int4b
    prob = synth.make_problem(M, N, K, dt, 128, seed=9)
    assert ops.plan(M, N, K, dt, 0, 128)["kernel"] == 1
    need = ops.workspace_bytes(M, N, K, dt, 0, 128)
    assert need > (1 << 20)  # room for 12 tile slabs of 256 x 128 fp32
    ws = torch.zeros(4096 if small_ws else need, dtype=torch.uint8, device=dev)
    bq = packing.interleave(prob["codes"], dt).to(dev)
    c = ops.quantized_matmul(prob["a"].to(dev), bq, prob["scales"].to(dev), dt, 128, 0, workspace=ws)
    torch.cuda.synchronize()
    assert int(ws.count_nonzero()) == 0, "workspace not restored to zero"
    ref = qo.quantized_matmul(prob["a"].numpy(), prob["codes"].numpy(), prob["scales"].numpy(), dt, 128, 0)
    got = c.cpu().numpy()
    assert _rel_err(got, ref) <= REL_TOL
    for n0 in range(0, N, 1024):  # the cut tiles are the last ones in raster order: look at every column range
        assert _rel_err(got[:, n0:n0 + 1024], ref[:, n0:n0 + 1024]) <= REL_TOL, n0


@pytest.mark.parametrize("M", [512, 4096, 4097])
def test_umma_kernel_many_row_tiles(M):
    """The persistent tile walk of the prefill kernel with more than one row tile, more tiles than
    SMs, row-tile groups (rasterisation) and - for 4097 - a last row tile of a single row that the
    activation copy fills with zeros (the reference benchmarks M = 4096 and 4097 itself,
    examples/quantization/matmul_a16wx.py:566-571).  Full comparison with the oracle."""
    N, K = 1024, 8192
    prob = synth.make_problem(M, N, K, D.int4b, 128, seed=M)
    pl = ops.plan(M, N, K, D.int4b, 0, 128)
    assert pl["kernel"] == 1 and pl["m_tiles"] > 1
    c, _, _ = _run(prob)
    ref = qo.quantized_matmul(prob["a"].numpy(), prob["codes"].numpy(), prob["scales"].numpy(), D.int4b, 128, 0)
    assert c.shape == (M, N)
    assert _rel_err(c, ref) <= REL_TOL
    # every row tile separately: a wrong tile cannot hide behind the largest element of the matrix
    for m0 in range(0, M, 256):
        assert _rel_err(c[m0:m0 + 256], ref[m0:m0 + 256]) <= REL_TOL, m0


def test_config2_prefill_full_size_sampled_columns():
    """BASELINE configuration 2 at full size: M = 4096, K = 8192, N = 28672, int4 g128, seed 0.  The
    oracle dequantizes and multiplies 512 sampled columns (every 128-column tile boundary region is
    hit: the stride 56 is coprime to 128); on the same columns the library's dequantized weights
    must be bit-identical."""
    dev = _dev()
    M, N, K = 4096, 28672, 8192
    prob = synth.make_problem(M, N, K, D.int4b, 128, seed=0)
    bq = packing.interleave(prob["codes"].to(dev), D.int4b)
    sc = prob["scales"].to(dev)
    a = prob["a"].to(dev)
    c = ops.quantized_matmul(a, bq, sc, D.int4b, 128, 0)
    cols = torch.arange(5, N, 56)[:512]
    w_cols = ops.dequantize(bq, sc, D.int4b, 128, 0)[:, cols.to(dev)].cpu().numpy()
    torch.cuda.synchronize()
    want_w = qo.dequantize(prob["codes"][:, cols].numpy(), prob["scales"][:, cols].numpy(), D.int4b, 128, 0)
    np.testing.assert_array_equal(w_cols.view(np.uint16), want_w.view(np.uint16))
    ref = qo.gemm_fp16(prob["a"].numpy(), want_w)
    got = c[:, cols.to(dev)].cpu().numpy()
    assert _rel_err(got, ref) <= REL_TOL
    for m0 in range(0, M, 1024):
        assert _rel_err(got[m0:m0 + 1024], ref[m0:m0 + 1024]) <= REL_TOL, m0


@pytest.mark.parametrize("M", [9, 12, 16])
@pytest.mark.parametrize("N,K", [(8192, 8192), (4096, 4096), (272, 14336)])
def test_stream_kernel_two_row_tiles_default_plan(M, N, K):
    """9..16 rows run the mma.sync kernel with two 8-row activation tiles, one CTA per SM: K in
    chunks, own tiles meeting in the fp32 scratch, left-over tiles (N = 272)."""
    prob = synth.make_problem(M, N, K, D.uint4b, 128, seed=M + N)
    assert ops.plan(M, N, K, D.uint4b, 8, 128)["kernel"] == 2
    c, _, _ = _run(prob)
    ref = qo.quantized_matmul(prob["a"].numpy(), prob["codes"].numpy(), prob["scales"].numpy(), D.uint4b, 128, 8)
    assert _rel_err(c, ref) <= REL_TOL


@pytest.mark.parametrize("M", [1, 16, 40, 200, 300])
@pytest.mark.parametrize("K,group", [(640, 128), (1152, 64), (1024, 32), (1152, 384), (2048, 64), (896, 896)])
@pytest.mark.parametrize("dt,zp", [(D.int4b, 0), (D.float6_e3m2, 0), (D.uint3b, 4)], ids=lambda x: getattr(x, "name", str(x)))
def test_gemm_general_k_and_small_groups(M, K, group, dt, zp):
    """The reference operator takes K % 16 == 0 and scale groups that are multiples of 32
    (examples/quantization/matmul_a16wx.py:66-71, :207).  Here: K any multiple of 128, groups of 32, 64
    or any multiple of 128.  What the decode kernel does not take (K not in whole 512-row blocks,
    groups below 128) runs on the tensor-core kernels for every M."""
    N = 272
    prob = synth.make_problem(M, N, K, dt, group, seed=K + group + M)
    prob["zero_point"] = zp
    c, bq, sc = _run(prob)
    want_w = qo.dequantize(prob["codes"].numpy(), prob["scales"].numpy(), dt, group, zp)
    if M == 1:  # the weights the kernels multiply by, bit for bit (general K layout, small groups)
        w = ops.dequantize(bq, sc, dt, group, zp).cpu().numpy()
        np.testing.assert_array_equal(w.view(np.uint16), want_w.view(np.uint16))
    ref = qo.gemm_fp16(prob["a"].numpy(), want_w)
    assert _rel_err(c, ref) <= REL_TOL


def test_config0_m16_k4096_n4096_u4():
    prob = synth.make_problem(16, 4096, 4096, D.uint4b, 128, seed=0)
    c, bq, sc = _run(prob)
    w = ops.dequantize(bq, sc, D.uint4b, 128, 8).cpu().numpy()
    want_w = qo.dequantize(prob["codes"].numpy(), prob["scales"].numpy(), D.uint4b, 128, 8)
    np.testing.assert_array_equal(w.view(np.uint16), want_w.view(np.uint16))
    ref = qo.gemm_fp16(prob["a"].numpy(), want_w)
    assert _rel_err(c, ref) <= REL_TOL


@pytest.mark.parametrize("dt", [D.uint1b, D.uint2b, D.uint3b, D.uint4b, D.uint6b, D.uint8], ids=lambda d: d.name)
def test_config1_decode_m1_k8192_n8192(dt):
    prob = synth.make_problem(1, 8192, 8192, dt, 128, seed=0)
    c, _, _ = _run(prob)
    ref = qo.quantized_matmul(prob["a"].numpy(), prob["codes"].numpy(), prob["scales"].numpy(), dt, 128,
                              prob["zero_point"])
    assert _rel_err(c, ref) <= REL_TOL


@pytest.mark.parametrize("dt", [D.float6_e3m2, D.int3b], ids=lambda d: d.name)
@pytest.mark.parametrize("M", [1, 4, 16, 64, 256])
def test_config3_per_channel(dt, M):
    K = N = 4096
    prob = synth.make_problem(M, N, K, dt, K, seed=0, scale_range=(0.5, 2.0))
    c, _, _ = _run(prob)
    ref = qo.quantized_matmul(prob["a"].numpy(), prob["codes"].numpy(), prob["scales"].numpy(), dt, K, 0)
    assert _rel_err(c, ref) <= REL_TOL


def test_linearity_full_size():
    """Size-independent property at full decode size: C(a1 + a2) == C(a1) + C(a2) up to
    fp16 output rounding, and scaling a column's scales by 2 doubles that column."""
    dev = _dev()
    N = K = 8192
    prob = synth.make_problem(2, N, K, D.uint4b, 128, seed=5)
    bq = packing.interleave(prob["codes"], D.uint4b).to(dev)
    sc = prob["scales"].to(dev)
    a = prob["a"].to(dev)
    a = (a * 0.25).to(torch.float16)
    a_sum = (a[0:1].float() + a[1:2].float()).to(torch.float16)
    c12 = ops.quantized_matmul(a, bq, sc, D.uint4b, 128, 8).float()
    cs = ops.quantized_matmul(a_sum, bq, sc, D.uint4b, 128, 8).float()
    torch.cuda.synchronize()
    scale_ref = c12.abs().max().item()
    assert (cs[0] - (c12[0] + c12[1])).abs().max().item() <= 1e-2 * scale_ref
    sc2 = sc.clone()
    sc2[:, ::2] *= 2
    c2 = ops.quantized_matmul(a, bq, sc2, D.uint4b, 128, 8).float()
    torch.cuda.synchronize()
    assert (c2[:, ::2] - 2 * c12[:, ::2]).abs().max().item() <= 4e-3 * scale_ref
    # untouched columns: equal up to the order of the fp32 split-K additions
    assert (c2[:, 1::2] - c12[:, 1::2]).abs().max().item() <= 2e-3 * scale_ref


def test_errors_are_loud():
    dev = _dev()
    prob = synth.make_problem(1, 64, 1024, D.uint4b, 128, seed=1)
    bq = packing.interleave(prob["codes"], D.uint4b).to(dev)
    with pytest.raises(Exception):
        ops.quantized_matmul(prob["a"], bq, prob["scales"].to(dev), D.uint4b, 128, 8)  # CPU activations
    with pytest.raises(Exception):
        ops.quantized_matmul(prob["a"].to(dev), bq, prob["scales"].to(dev), D.uint4b, 128, 3)  # bad zero point
    small_ws = torch.zeros(256, dtype=torch.uint8, device=dev)
    with pytest.raises(Exception):
        ops.quantized_matmul(prob["a"].to(dev), bq, prob["scales"].to(dev), D.uint4b, 128, 8, workspace=small_ws)
