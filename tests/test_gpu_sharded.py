"""Column-sharded layers with the all-gather fused into the GEMV kernel (b200q_gemm_gather).

One GPU is enough: the ranks of a two-rank group are played one after the other on one stream, with
both ranks' row buffers and flags in this process's memory, so the kernel's addressing (column
offsets, every rank's buffer, buffer alternation) and its flag protocol (wait for the previous
epoch, raise the own slot everywhere) run exactly as they do across GPUs - only the transport
(peer-mapped pointers over NVLink) is not exercised here."""
import numpy as np
import pytest
import torch

from oracle import quant_oracle as qo
from tilus_b200 import _lib, float16, ops, sharded, synth
from tilus_b200 import dtypes as D

pytestmark = pytest.mark.gpu


def _virtual_group(world, max_rows, max_cols, dev, tagged_rows=0):
    """tagged_rows = 0: every fused call uses the flag protocol; n: batches of up to n rows use tagged words"""
    regions = [torch.zeros(sharded.PeerGather.region_bytes(max_rows, max_cols, tagged_rows), dtype=torch.uint8,
                           device=dev) for _ in range(world)]
    ptrs = [r.data_ptr() for r in regions]
    return regions, [sharded.PeerGather(world, r, ptrs, max_rows, max_cols, dev, tagged_rows) for r in range(world)]


@pytest.mark.parametrize("tagged", [False, True], ids=["flags", "tagged"])
@pytest.mark.parametrize("M", [1, 5, 16])
@pytest.mark.parametrize("world", [2, 4])
def test_fused_gather_chain_matches_unsharded(M, world, tagged):
    dev = torch.device("cuda:0")
    dt, g = D.uint4b, 128
    dims = [(1024, 2048), (2048, 1024), (1024, 512)]  # a chain of three layers
    probs = [synth.make_problem(M, n, k, dt, g, seed=10 + i) for i, (k, n) in enumerate(dims)]
    regions, ctxs = _virtual_group(world, 16, 2048, dev, 16 if tagged else 0)
    shards = []
    for (k, n), prob in zip(dims, probs):
        per_rank = []
        for r in range(world):
            lin = sharded.ShardedQuantizedLinear(float16, dt, g, k, n, zero_point=prob["zero_point"],
                                                 shard=(world, r)).to(dev)
            lin.load_codes(prob["codes"], prob["scales"])
            per_rank.append(lin)
        shards.append(per_rank)
    x0 = (probs[0]["a"] * 0.25).to(torch.float16).to(dev)
    xs = [x0 for _ in range(world)]
    for per_rank in shards:  # one fused call per layer; the ranks take their turns on one stream
        xs = [ctxs[r].gemm(xs[r], per_rank[r]) for r in range(world)]
    outs = [ctxs[r].fetch(xs[r]) for r in range(world)]
    # reference: the same chain through the oracle, fp16 between layers
    ref = x0.cpu().numpy()
    for (k, n), prob in zip(dims, probs):
        ref = qo.quantized_matmul(ref, prob["codes"].numpy(), prob["scales"].numpy(), dt, g, prob["zero_point"])
    for r in range(world):
        got = outs[r].float().cpu().numpy()
        assert got.shape == (M, dims[-1][1])
        err = np.abs(got - ref.astype(np.float32)).max() / np.abs(ref.astype(np.float32)).max()
        assert err <= 2e-2, (r, err)  # three layers deep: tolerance of the single GEMM, doubled
    # every rank saw every rank finish the last call, and counted its own calls
    for r in range(world):
        flags = regions[r][: 4 * world].view(torch.int32).cpu().numpy()
        assert (flags == (0 if tagged else len(dims))).all()
        assert ctxs[r].calls_completed(tagged) == len(dims)
        assert ctxs[r].calls_completed(not tagged) == 0
    assert ops.device_status(ops.get_workspace(dev, 1 << 20)) == [0, 0, 0, 0]


@pytest.mark.parametrize("tagged", [False, True], ids=["flags", "tagged"])
def test_fused_gather_replays_from_a_cuda_graph(tagged):
    """The calls carry no per-call state: a captured chain can be replayed and keeps counting."""
    dev = torch.device("cuda:0")
    dt, g, M, world = D.int4b, 128, 2, 2
    prob = synth.make_problem(M, 1024, 1024, dt, g, seed=3)
    regions, ctxs = _virtual_group(world, 16, 1024, dev, 2 if tagged else 0)
    lins = []
    for r in range(world):
        lin = sharded.ShardedQuantizedLinear(float16, dt, g, 1024, 1024, shard=(world, r)).to(dev)
        lin.load_codes(prob["codes"], prob["scales"])
        lins.append(lin)
    x = (prob["a"] * 0.25).to(torch.float16).to(dev)

    def chain():
        rows = [ctxs[r].gemm(x, lins[r]) for r in range(world)]          # call 1: external activations
        return [ctxs[r].gemm(rows[r], lins[r]) for r in range(world)]     # call 2: previous output

    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        rows = chain()  # warm-up (sets kernel attributes, allocates the workspace)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            rows = chain()
        for _ in range(3):
            graph.replay()
        want1 = qo.quantized_matmul(x.cpu().numpy(), prob["codes"].numpy(), prob["scales"].numpy(), dt, g, 0)
        want2 = qo.quantized_matmul(want1, prob["codes"].numpy(), prob["scales"].numpy(), dt, g, 0)
        for r in range(world):
            assert ctxs[r].calls_completed(tagged) == 2 + 3 * 2
            got = ctxs[r].fetch(rows[r]).float().cpu().numpy()
            err = np.abs(got - want2.astype(np.float32)).max() / np.abs(want2.astype(np.float32)).max()
            assert err <= 2e-2


def test_fused_gather_rejects_wide_batches():
    dev = torch.device("cuda:0")
    regions, ctxs = _virtual_group(2, 16, 512, dev)
    lin = sharded.ShardedQuantizedLinear(float16, D.int4b, 128, 512, 512, shard=(2, 0)).to(dev)
    prob = synth.make_problem(1, 512, 512, D.int4b, 128, seed=1)
    lin.load_codes(prob["codes"], prob["scales"])
    with pytest.raises(ValueError):
        ctxs[0].gemm(torch.zeros(17, 512, dtype=torch.float16, device=dev), lin)


@pytest.mark.parametrize("M", [9, 12])
def test_fused_gather_wide_shard_workspace(M):
    """9..16 rows with a wide shard: the workspace b200q_workspace_bytes reports for the problem (fp32
    scratch [N_loc][16]) is what the fused call needs - here more than the 1 MiB the operator layer
    allocates at least."""
    dev = torch.device("cuda:0")
    dt, g, world = D.uint4b, 128, 2
    K, N = 512, 2 * 28672
    prob = synth.make_problem(M, N, K, dt, g, seed=M)
    need = ops.workspace_bytes(M, N // world, K, dt, prob["zero_point"], g)
    assert need > (1 << 20)
    regions, ctxs = _virtual_group(world, 16, N, dev)
    rows = []
    for r in range(world):
        lin = sharded.ShardedQuantizedLinear(float16, dt, g, K, N, zero_point=prob["zero_point"], shard=(world, r)).to(dev)
        lin.load_codes(prob["codes"], prob["scales"])
        rows.append(ctxs[r].gemm(prob["a"].to(dev), lin))
    ref = qo.quantized_matmul(prob["a"].numpy(), prob["codes"].numpy(), prob["scales"].numpy(), dt, g,
                              prob["zero_point"]).astype(np.float32)
    for r in range(world):
        got = ctxs[r].fetch(rows[r]).float().cpu().numpy()
        assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-2


def test_fused_gather_wait_runs_out_and_reports():
    """A bounded device-side wait that runs out: rank 0 of a two-rank group makes two fused calls while
    rank 1 makes none, so rank 0's second launch waits for a flag that nothing raises.  After a
    quarter of a second it gives up, completes normally and leaves B200Q_ERR_DEVICE_TIMEOUT with the
    place (5 = wait for a peer's columns) in the workspace header; reading the status clears it, and
    the context stays usable."""
    dev = torch.device("cuda:0")
    dt, g, M = D.int4b, 128, 2
    prob = synth.make_problem(M, 512, 512, dt, g, seed=4)
    regions, ctxs = _virtual_group(2, 16, 512, dev)
    lin = sharded.ShardedQuantizedLinear(float16, dt, g, 512, 512, shard=(2, 0)).to(dev)
    lin.load_codes(prob["codes"], prob["scales"])
    x = prob["a"].to(dev)
    ws = ops.get_workspace(dev, ops.workspace_bytes(M, 256, 512, dt, 0, g))
    assert ops.device_status(ws) == [0, 0, 0, 0]
    ctxs[0].gemm(x, lin)  # call 1: nothing to wait for
    assert ops.device_status(ws) == [0, 0, 0, 0]
    ctxs[0].gemm(x, lin)  # call 2: rank 1 never finished call 1
    torch.cuda.synchronize()
    st = ops.device_status(ws)
    assert st[0] == _lib.ST_DEVICE_TIMEOUT and st[1] == 5, st
    assert ops.device_status(ws) == [0, 0, 0, 0]  # reading cleared the report
    assert ctxs[0].calls_completed() == 2          # the launch ran to its end
    # the library still computes: an ordinary GEMM on the same workspace right after
    assert int(ws.count_nonzero()) == 0
    c = ops.quantized_matmul(x, lin.local.quantized_weight.data, lin.local.scales.data, dt, g, 0, workspace=ws)
    ref = qo.quantized_matmul(prob["a"].numpy(), prob["codes"][:, :256].numpy(), prob["scales"][:, :256].numpy(), dt, g, 0)
    err = np.abs(c.float().cpu().numpy() - ref.astype(np.float32)).max() / np.abs(ref.astype(np.float32)).max()
    assert err <= 1e-2


def test_tagged_gather_wait_runs_out_and_reports():
    """The same with tagged words: rank 0's second call reads the previous call's rows, of which rank 1's
    half never arrived; the loads of those words give up after a quarter of a second."""
    dev = torch.device("cuda:0")
    dt, g, M = D.int4b, 128, 2
    prob = synth.make_problem(M, 512, 512, dt, g, seed=4)
    regions, ctxs = _virtual_group(2, 16, 512, dev, 2)
    lin = sharded.ShardedQuantizedLinear(float16, dt, g, 512, 512, shard=(2, 0)).to(dev)
    lin.load_codes(prob["codes"], prob["scales"])
    ws = ops.get_workspace(dev, ops.workspace_bytes(M, 256, 512, dt, 0, g))
    assert ops.device_status(ws) == [0, 0, 0, 0]
    row = ctxs[0].gemm(prob["a"].to(dev), lin)  # call 1: activations from outside, nothing to wait for
    torch.cuda.synchronize()
    assert ops.device_status(ws) == [0, 0, 0, 0]
    ctxs[0].gemm(row, lin)                      # call 2: columns 256.. of call 1's row never arrive
    torch.cuda.synchronize()
    st = ops.device_status(ws)
    assert st[0] == _lib.ST_DEVICE_TIMEOUT and st[1] == 5, st
    assert ops.device_status(ws) == [0, 0, 0, 0]
    assert ctxs[0].calls_completed(True) == 2
    assert int(ws.count_nonzero()) == 0


@pytest.mark.parametrize("M", [1, 12])
def test_tagged_gather_bf16_chain(M):
    """bfloat16 activations through the tagged hand-over: two chained layers on a two-rank group against
    the bf16 oracle (rows handed over as bf16 pairs with their tags)."""
    from tilus_b200 import bfloat16

    dev = torch.device("cuda:0")
    dt, g, world = D.int4b, 128, 2
    dims = [(1024, 2048), (2048, 512)]
    probs = [synth.make_problem(M, n, k, dt, g, seed=50 + i) for i, (k, n) in enumerate(dims)]
    regions, ctxs = _virtual_group(world, 16, 2048, dev, 16)
    x0 = (probs[0]["a"] * 0.25).to(torch.bfloat16)
    xs = [x0.to(dev)] * world
    ref = x0
    for (k, n), prob in zip(dims, probs):
        lins = []
        for r in range(world):
            lin = sharded.ShardedQuantizedLinear(bfloat16, dt, g, k, n, shard=(world, r)).to(dev)
            lin.load_codes(prob["codes"], prob["scales"].to(torch.bfloat16))
            lins.append(lin)
        xs = [ctxs[r].gemm(xs[r], lins[r]) for r in range(world)]
        ref = qo.quantized_matmul_bf16(ref, prob["codes"].numpy(), prob["scales"].to(torch.bfloat16), dt, g, 0)
    want = ref.float().numpy()
    for r in range(world):
        got = ctxs[r].fetch(xs[r])
        assert got.dtype == torch.bfloat16
        err = np.abs(got.float().cpu().numpy() - want).max() / np.abs(want).max()
        assert err <= 2e-2, (r, err)
        assert ctxs[r].calls_completed(True) == len(dims)


def test_tagged_gather_two_outside_calls_in_a_row():
    """Two tagged calls in a row that take their activations from outside: the context puts a wait for
    the first one's rows between them (the rule of the tagged mode), and results stay right."""
    dev = torch.device("cuda:0")
    dt, g, M, world = D.uint4b, 128, 1, 2
    prob = synth.make_problem(M, 1024, 512, dt, g, seed=8)
    regions, ctxs = _virtual_group(world, 16, 1024, dev, 2)
    lins = []
    for r in range(world):
        lin = sharded.ShardedQuantizedLinear(float16, dt, g, 512, 1024, zero_point=prob["zero_point"], shard=(world, r)).to(dev)
        lin.load_codes(prob["codes"], prob["scales"])
        lins.append(lin)
    x = prob["a"].to(dev)
    ref = qo.quantized_matmul(prob["a"].numpy(), prob["codes"].numpy(), prob["scales"].numpy(), dt, g,
                              prob["zero_point"]).astype(np.float32)
    for _ in range(4):
        rows = [ctxs[r].gemm(x, lins[r]) for r in range(world)]
    for r in range(world):
        got = ctxs[r].fetch(rows[r]).float().cpu().numpy()
        assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-2
        assert ctxs[r].calls_completed(True) == 4
    assert ops.device_status(ops.get_workspace(dev, 1 << 20)) == [0, 0, 0, 0]


@pytest.mark.parametrize("tagged", [False, True], ids=["flags", "tagged"])
@pytest.mark.parametrize("M", [20, 64])
def test_push_collect_gather_above_16_rows(M, tagged):
    """More than 16 rows: local GEMM, then push (shard to every rank's row buffer + flags) and collect
    (wait for all shards, copy the rows out).  Two ranks played on one stream: both push, then both
    collect - a collect waits for the pushes of the same call, so they must all have been queued."""
    dev = torch.device("cuda:0")
    dt, g, world = D.int4b, 128, 2
    dims = [(512, 1024), (1024, 512)]
    probs = [synth.make_problem(M, n, k, dt, g, seed=30 + i) for i, (k, n) in enumerate(dims)]
    regions, ctxs = _virtual_group(world, 64, 1024, dev, 64 if tagged else 0)
    x = [(probs[0]["a"] * 0.25).to(torch.float16).to(dev)] * world
    ref = x[0].cpu().numpy()
    for (k, n), prob in zip(dims, probs):
        lins = []
        for r in range(world):
            lin = sharded.ShardedQuantizedLinear(float16, dt, g, k, n, shard=(world, r)).to(dev)
            lin.load_codes(prob["codes"], prob["scales"])
            lins.append(lin)
        shards = [lins[r].local(x[r]) for r in range(world)]
        for r in range(world):
            ctxs[r].push(shards[r], lins[r], tagged)
        full = [torch.empty(M, n, dtype=torch.float16, device=dev) for _ in range(world)]
        for r in range(world):
            ctxs[r].collect(full[r], M, n, tagged)
        x = full
        ref = qo.quantized_matmul(ref, prob["codes"].numpy(), prob["scales"].numpy(), dt, g, 0)
    torch.cuda.synchronize()
    ws = ops.get_workspace(dev, 1 << 20)
    assert ops.device_status(ws) == [0, 0, 0, 0]
    for r in range(world):
        got = x[r].float().cpu().numpy()
        err = np.abs(got - ref.astype(np.float32)).max() / np.abs(ref.astype(np.float32)).max()
        assert err <= 2e-2, (r, err)
        assert ctxs[r].calls_completed(tagged) == len(dims)
