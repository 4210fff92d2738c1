"""Benchmark of the weight-only quantized matmul hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--no-sweep] [--no-prefill] [--no-stack] [--stack]
                    [--profile-case decode|prefill|batch16|batch32]

Headline workload (one GPU): decode GEMV, M=1, K=N=8192, uint4 codes with zero point 8,
group 128, fp16 scales - the "u4 g128" decode configuration the metric is quoted on.
One step = ROUNDS passes over R distinct layers of that shape (R * weights > L2, so every
launch streams its weights from HBM); the R * ROUNDS launches are replayed from one CUDA
graph.  `value` is algorithmic GB/s: (packed weights + scales + activations + output)
bytes of all launches divided by the device time of the timed region.  With N > 1 GPUs
every rank runs the same per-GPU workload on its own column shard (weak scaling, no
collective on the data path) and `value` is the aggregate.

The JSON line also carries: `roofline` (HBM, for the GEMV kernel), `e2e` (same metric
through QuantizedLinear.forward with pinned host activations copied in and the result
copied out every step), `cpu_baseline` (the CPU oracle - the reference's PyTorch
dequantize + matmul semantics - timed on this host), `clocks`, `gpu_launches`,
`headline_shapes` (the metric's three shapes M = 1 / 16 / 4096 against their rooflines),
`stack` (the Llama-3-8B-shaped decode linear stack, N-sharded over the ranks of this run
with an all-gather per layer: NCCL and over peer memory - fused into the GEMV kernel for
M <= 16, a push / collect kernel pair above -, strong scaling) and an
`extra` sweep: the other bit widths at M=1, M=16, the M=16 K=N=4096 configuration, the
per-channel float6 / int3 batch sweep, the Llama-3-8B layer shapes at M in {1, 8, 32, 64},
the reference example's own table (K=4096, N=12288, eight weight types, M in {1, 16, 4096,
4097}) and the M=4096 prefill GEMM in TFLOP/s.  Every sweep entry is checked against the
oracle on sampled columns (`rel_err`).

`--impl reference` times the CPU dequantize + matmul path alone (the reference operator's
semantics on the host cores), on the same workload and metric.

`--stack` runs only the Llama-3-8B-shaped decode linear stack (the `stack` entry of the main
line) and prints it as a line of its own.

`--profile-case X` runs a few plain launches of one kernel on a problem larger than L2 and
prints its CUDA-event time: the command line used for the ncu captures under profiles/.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

M, K, N, GROUP, NBITS = 1, 8192, 8192, 128, 4
WORKLOAD = "decode_gemv_u4_g128_M1_K8192_N8192"
METRIC = "quant-GEMM HBM GB/s (u4 g128, M=1, K=N=8192)"
R_LAYERS = 10   # distinct layers per pass: 10 x 33.5 MB of weights = 335 MB > 126 MB L2
ROUNDS = 10     # passes per graph: 100 launches per replay


def _decode_dram_traffic():
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the headline kernel, as recorded
    with the ncu capture it came from (None when no capture is on record)."""
    path = os.path.join(ROOT, "profiles", "decode_dram_traffic.json")
    try:
        with open(path) as f:
            return json.load(f)
    except (OSError, ValueError):
        return None


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), tflops=float(p.get("bf16_tflops", 0.0)),
                    tflops_sustained=float(p.get("bf16_tflops_sustained", 0.0)), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def _cpu_gemv_seconds(prob, repeats: int, warm: bool = True) -> float:
    """The oracle's dequantize + matmul (reference semantics) on the host cores: seconds per call."""
    from oracle import quant_oracle as qo

    torch.set_num_threads(os.cpu_count() or 1)
    a, codes, scales = prob["a"].numpy(), prob["codes"].numpy(), prob["scales"].numpy()
    if warm:
        qo.quantized_matmul(a, codes, scales, prob["dtype"], prob["group_size"], prob["zero_point"])
    t0 = time.perf_counter()
    for _ in range(repeats):
        qo.quantized_matmul(a, codes, scales, prob["dtype"], prob["group_size"], prob["zero_point"])
    return (time.perf_counter() - t0) / repeats


def run_reference(args) -> None:
    from tilus_b200 import dtypes, synth

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    prob = synth.make_problem(M, N, K, dtypes.uint4b, GROUP, seed=0)
    nbytes = synth.gemm_bytes(M, N, K, NBITS, GROUP)
    _cpu_gemv_seconds(prob, max(args.warmup, 1), warm=False)      # warm-up steps: one oracle call each
    dt = _cpu_gemv_seconds(prob, args.steps, warm=False)          # a step = one oracle call
    val = nbytes / dt / 1e9
    cores = os.cpu_count() or 1
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": "n/a (CPU)"},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": "one full M=1 K=N=8192 u4 g128 dequantize+matmul per step (oracle, torch CPU)"},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def _time_graph(graph, reps: int) -> float:
    """Device milliseconds of `reps` replays, CUDA events on the current stream."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def _make_layers(dt, n, k, group, count, dev, seed=0, scale_range=(0.005, 0.02), distinct=True, prob0=None):
    """`count` QuantizedLinear layers [k -> n] on the device.  distinct=False generates one
    synthetic problem (or takes `prob0`) and gives every layer its own copy of it (same timing,
    faster set-up)."""
    from tilus_b200 import QuantizedLinear, float16, synth

    layers = []
    first = None
    for i in range(count):
        if distinct or first is None:
            prob = prob0 if (prob0 is not None and not distinct) else \
                synth.make_problem(1, n, k, dt, group, seed=seed + i, scale_range=scale_range)
            layer = QuantizedLinear(float16, dt, group, k, n, zero_point=prob["zero_point"]).to(dev)
            layer.load_codes(prob["codes"].to(dev), prob["scales"].to(dev))
            if first is None:
                first = layer
        else:
            layer = QuantizedLinear(float16, dt, group, k, n, zero_point=first.zero_point).to(dev)
            layer.load_packed(first.quantized_weight.data.clone(), first.scales.data.clone(), layout="b200")
        layers.append(layer)
    return layers


def _acts(m, k, count, dev, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(m, k, generator=g, dtype=torch.float32).to(torch.float16).to(dev) for _ in range(count)]


def _capture(layers, acts, rounds=1):
    outs = [None] * len(layers)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm on the capture stream: its workspace exists before capture
        for layer, a in zip(layers, acts):
            layer(a)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for _ in range(rounds):
            for i, (layer, a) in enumerate(zip(layers, acts)):
                outs[i] = layer(a)
    return g, outs


def _layer_count(dt, n, k):
    """Enough layers that one pass streams more than 300 MiB of weights (> L2)."""
    wbytes = k * n * dt.nbits // 8
    return max(2, min(40, (300 * 2**20 + wbytes - 1) // wbytes))


def _spot_check(prob, a_cpu, got, cols) -> float:
    """rel-err of the kernel's output against the oracle on sampled columns."""
    from oracle import quant_oracle as qo

    ref = qo.quantized_matmul(a_cpu.numpy(), prob["codes"][:, cols].numpy(), prob["scales"][:, cols].numpy(),
                              prob["dtype"], prob["group_size"], prob["zero_point"]).astype("float32")
    out = got[:, cols.to(got.device)].float().cpu().numpy()
    return float(abs(out - ref).max() / max(abs(ref).max(), 1e-30))


def _sweep_shape(dt, n, k, group, ms_list, dev, reps, scale_range=(0.005, 0.02)):
    """us / GB/s / TFLOP/s of one layer shape for each M, layers rotated so weights stream from HBM.
    All layers of a shape hold the same synthetic weights (own copies, so the bytes still stream
    from HBM); what was timed is compared with the oracle on 64 sampled columns."""
    from tilus_b200 import synth

    count = _layer_count(dt, n, k)
    prob = synth.make_problem(1, n, k, dt, group, seed=100, scale_range=scale_range)
    layers = _make_layers(dt, n, k, group, count, dev, seed=100, scale_range=scale_range, distinct=False, prob0=prob)
    cols = torch.arange(3, n, max(1, n // 64))[:64]
    out = {}
    for m in ms_list:
        acts = _acts(m, k, count, dev, seed=m)
        rounds = max(1, 40 // count) if m <= 64 else 1
        g, outs = _capture(layers, acts, rounds)
        _time_graph(g, 3)
        ms = _time_graph(g, reps) / (reps * count * rounds)
        nbytes = synth.gemm_bytes(m, n, k, dt.nbits, group)
        out[m] = {"us": ms * 1e3, "gbs": nbytes / (ms * 1e-3) / 1e9,
                  "tflops": synth.gemm_flops(m, n, k) / (ms * 1e-3) / 1e12,
                  "rel_err": _spot_check(prob, acts[0].cpu(), outs[0], cols)}
        del g, acts, outs
    del layers
    torch.cuda.empty_cache()
    return out


def _sweep_followers(dev, hbm) -> dict:
    """The rows the path was widened into: bfloat16 activations on the headline shape, and the gate_up
    projection with SwiGLU and the per-token FP8 cast behind it (one library call), each checked against
    its oracle on what was timed."""
    from oracle import cast_oracle as co
    from oracle import quant_oracle as qo
    from tilus_b200 import QuantizedLinear, bfloat16, dtypes, ops, packing, synth

    out = {}
    dt = dtypes.uint4b
    # ---- bf16 activations, decode GEMV M = 1, K = N = 8192 ----
    n = k = 8192
    prob = synth.make_problem(1, n, k, dt, GROUP, seed=100)
    count = _layer_count(dt, n, k)
    bq = packing.interleave(prob["codes"].to(dev), dt)
    sc = prob["scales"].to(torch.bfloat16).to(dev)
    layers = []
    for _ in range(count):
        layer = QuantizedLinear(bfloat16, dt, GROUP, k, n, zero_point=prob["zero_point"]).to(dev)
        layer.load_packed(bq.clone(), sc.clone(), layout="b200")
        layers.append(layer)
    acts = [a.to(torch.bfloat16) for a in _acts(1, k, count, dev, seed=1)]
    rounds = max(1, 40 // count)
    g, outs = _capture(layers, acts, rounds)
    _time_graph(g, 3)
    ms = _time_graph(g, 10) / (10 * count * rounds)
    cols = torch.arange(3, n, n // 64)[:64]
    ref = qo.quantized_matmul_bf16(acts[0].cpu(), prob["codes"][:, cols].numpy(), prob["scales"][:, cols].to(torch.bfloat16),
                                   dt, GROUP, prob["zero_point"]).float().numpy()
    got = outs[0][:, cols.to(dev)].float().cpu().numpy()
    nbytes = synth.gemm_bytes(1, n, k, dt.nbits, GROUP)
    out["bf16_decode_u4_M1_K8192_N8192"] = {
        "us": round(ms * 1e3, 3), "gbs": round(nbytes / (ms * 1e-3) / 1e9, 1),
        "hbm_frac": round(nbytes / (ms * 1e-3) / 1e9 / hbm, 4),
        "rel_err": float(f"{abs(got - ref).max() / max(abs(ref).max(), 1e-30):.3g}")}
    del g, outs, layers, acts
    torch.cuda.empty_cache()
    # ---- gate_up (K = 4096, N = 2 x 14336) + SwiGLU + per-token FP8 cast, M = 8, one call per layer ----
    k, n, m = 4096, 28672, 8
    prob = synth.make_problem(m, n, k, dt, GROUP, seed=101)
    count = _layer_count(dt, n, k)
    layers = _make_layers(dt, n, k, GROUP, count, dev, seed=101, distinct=False, prob0=prob)
    acts = _acts(m, k, count, dev, seed=2)
    res = [None] * count
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i, (layer, a) in enumerate(zip(layers, acts)):
            res[i] = layer.forward_swiglu_cast(a)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for i, (layer, a) in enumerate(zip(layers, acts)):
            res[i] = layer.forward_swiglu_cast(a)
    _time_graph(g, 3)
    ms = _time_graph(g, 10) / (10 * count)
    q, sf, gate_up = res[0]
    want_codes, want_sf, _ = co.swiglu_forward_and_per_token_cast(gate_up.float().cpu().numpy(), group=128)
    deq = q.float().cpu().numpy().reshape(m, -1, 128) * sf.cpu().numpy()[:, :, None]
    want = co.e4m3_decode(want_codes).astype("float32").reshape(m, -1, 128) * want_sf[:, :, None]
    out["gate_up_swiglu_fp8_cast_u4_M8_K4096_N28672"] = {
        "us": round(ms * 1e3, 3),
        "gemm_rel_err": float(f"{_spot_check(prob, acts[0].cpu(), gate_up, torch.arange(3, n, n // 64)[:64]):.3g}"),
        "cast_scale_max_abs_diff": float(f"{abs(sf.cpu().numpy() - want_sf).max():.3g}"),
        "cast_dequantized_rel_err": float(f"{abs(deq - want).max() / max(abs(want).max(), 1e-30):.3g}")}
    del g, res, layers, acts
    torch.cuda.empty_cache()
    return out


def run_profile_case(args) -> None:
    """A few plain (non-graph) launches of one kernel on inputs larger than L2."""
    from tilus_b200 import dtypes

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    case = args.profile_case
    if case == "decode":
        dt, m, n, k, count = dtypes.uint4b, 1, 8192, 8192, 6
    elif case == "batch16":
        dt, m, n, k, count = dtypes.uint4b, 16, 8192, 8192, 6
    elif case == "batch32":
        dt, m, n, k, count = dtypes.uint4b, 32, 8192, 8192, 6
    elif case == "prefill":
        dt, m, n, k, count = dtypes.int4b, 4096, 7168, 8192, 2
    else:
        raise SystemExit(f"unknown profile case {case}")
    layers = _make_layers(dt, n, k, GROUP, count, dev, seed=0, distinct=False)
    acts = _acts(m, k, count, dev)
    for _ in range(2):
        for layer, a in zip(layers, acts):
            layer(a)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for layer, a in zip(layers, acts):
        layer(a)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / count
    print(json.dumps({"profile_case": case, "dtype": dt.name, "M": m, "N": n, "K": k, "launches": 3 * count,
                      "us_per_launch_plain_stream": us}))


def measure_stack(world, rank, dev, steps, warmup, batches=(1, 8, 32, 64), tagged_rows=16) -> dict:
    """Llama-3-8B-shaped decode linear stack, N-sharded over the ranks, all-gather of every layer's
    output: 32 x {qkv 4096->6144, o 4096->4096, gate_up 4096->28672, down 14336->4096}, uint4 g128
    weights, batch M in {1, 8, 32, 64}.  Strong scaling: the model is fixed, the shards shrink with the
    number of ranks.  A step = one pass over the 128 linears, replayed from one CUDA graph.  Two forms
    of the all-gather: `nccl` (a collective per layer) and - for M <= 16 - `fused` (the GEMV kernel
    stores its columns into every rank's row buffer over NVLink and raises flags).  Before timing the
    fused rows are compared with the NCCL path's and, for the first block of four linears, both with
    the oracle.  The process group must be up when world > 1."""
    import torch.distributed as dist

    from oracle import quant_oracle as qo
    from tilus_b200 import dtypes, float16, packing, sharded, synth

    dt = dtypes.uint4b
    shapes = [("qkv", 4096, 6144), ("o", 4096, 4096), ("gate_up", 4096, 28672), ("down", 14336, 4096)]
    n_layers = 32
    protos, probs = {}, {}
    for name, k_in, n_out in shapes:  # one synthetic weight per shape, one device copy per layer
        # Values chosen so that the activations keep their magnitude through all 128 linears and the
        # comparisons below mean something: codes uniform in 1..15 (zero mean after the zero point 8;
        # uniform 0..15 has mean -0.5, a common mode that grows ~7x per layer) and scales around
        # 1 / (sqrt(K) * std(q - 8)).  The benchmark's own U(0.005, 0.02) scales overflow fp16 within a
        # few blocks; the timing does not depend on the values.
        s_mean = 1.0 / (k_in ** 0.5 * 4.32)
        prob = synth.make_problem(1, n_out, k_in, dt, GROUP, seed=7, scale_range=(0.75 * s_mean, 1.25 * s_mean))
        prob["codes"] = torch.randint(1, 16, (k_in, n_out), generator=torch.Generator().manual_seed(11),
                                      dtype=torch.int32).to(torch.uint8)
        probs[name] = prob
        n0, n1 = sharded.shard_range(n_out, world, rank)
        protos[name] = (packing.interleave(prob["codes"][:, n0:n1].contiguous().to(dev), dt),
                        prob["scales"][:, n0:n1].contiguous().to(dev), prob["zero_point"])
    layers = []
    for _ in range(n_layers):
        block = []
        for name, k_in, n_out in shapes:
            bq, sc, zp = protos[name]
            lin = sharded.ShardedQuantizedLinear(float16, dt, GROUP, k_in, n_out, zero_point=zp).to(dev)
            lin.local.load_packed(bq, sc, layout="b200")
            block.append(lin)
        layers.append(block)
    del protos
    weight_bytes = sum(k * n // 2 + (k // GROUP) * n * 2 for _, k, n in shapes) * n_layers // world

    def step(x, blocks=layers):
        for qkv, o, gate_up, down in blocks:
            h = qkv(x)
            h = o(h[:, :4096])
            h = gate_up(h)
            x = down(h[:, :14336])
        return x

    ctx = sharded.PeerGather.create(64, 28672, dev, tagged_rows=tagged_rows)

    def step_fused(x, blocks=layers):
        row = x
        for qkv, o, gate_up, down in blocks:
            row = ctx.gemm(row, qkv)
            row = ctx.gemm(ctx.cols(row, 0, 4096), o)
            row = ctx.gemm(row, gate_up)
            row = ctx.gemm(ctx.cols(row, 0, 14336), down)
        return row

    w_ref = {}

    def oracle_block(x_cpu):  # the first block of four linears, fp16 between them
        def mm(name, h):
            if name not in w_ref:
                pr = probs[name]
                w_ref[name] = qo.dequantize(pr["codes"].numpy(), pr["scales"].numpy(), dt, GROUP, pr["zero_point"])
            return qo.gemm_fp16(h, w_ref[name])

        h = mm("qkv", x_cpu.numpy())[:, :4096]
        h = mm("o", np.ascontiguousarray(h))
        h = mm("gate_up", h)[:, :14336]
        return mm("down", np.ascontiguousarray(h)).astype("float32")

    def rel(a, b):
        return float(abs(a - b).max() / max(abs(b).max(), 1e-30))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    results, graphs = {}, []
    for m in batches:
        x = (torch.randn(m, 4096, generator=torch.Generator().manual_seed(m)) * 0.05).to(torch.float16).to(dev)
        modes = ["nccl" if world > 1 else "single"] + ["fused"]
        entry = {}
        # ---- correctness of what is timed (all device work first: a rank that computed the oracle
        # in between would keep its peers' fused kernels waiting beyond their bounded wait) ----
        barrier()
        y_nccl = step(x).float().cpu().numpy()                      # full stack, NCCL gather
        y_blk = step(x, layers[:1]).float().cpu().numpy()           # first block
        if "fused" in modes:
            barrier()
            y_fused = ctx.fetch(step_fused(x)).float().cpu().numpy()
            y_fblk = ctx.fetch(step_fused(x, layers[:1])).float().cpu().numpy()
            entry["fused_vs_nccl_rel_err"] = rel(y_fused, y_nccl)
        barrier()
        if rank == 0:
            want = oracle_block(x.cpu())
            entry["block_vs_oracle_rel_err"] = rel(y_blk, want)
            if "fused" in modes:
                entry["fused_block_vs_oracle_rel_err"] = rel(y_fblk, want)
        barrier()
        for mode in modes:
            fn = step_fused if mode == "fused" else step
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn(x)
            barrier()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                fn(x)
            graphs.append(g)
            for _ in range(max(warmup, 3)):
                g.replay()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            entry[mode] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(m / (ms * 1e-3), 1),
                           "us_per_linear": round(ms * 1e3 / (4 * n_layers), 2),
                           "per_gpu_weight_gbs": round(weight_bytes / (ms * 1e-3) / 1e9, 1)}
            barrier()
        results[f"M{m}"] = entry
    # graphs that captured collectives go before the communicator does
    for g in graphs:
        g.reset()
    del graphs
    barrier()
    ctx.close()
    return {"workload": "llama3_8b_linear_stack_u4_g128", "layers": n_layers, "linears_per_step": 4 * n_layers,
            "scaling": "strong", "unit": "ms per 128-linear step", "per_gpu_weight_bytes": weight_bytes,
            "gather": {"nccl": "ncclAllGather per layer (M > 1: + one permute copy)",
                       "fused": f"M <= {tagged_rows} on 2+ GPUs: rows handed over as tagged words, polled by the next "
                                "kernel (b200q_gemm_gather / b200q_gather_push, B200Q_GATHER_TAGGED), else per-rank flags; "
                                "M <= 16: peer stores from the GEMV kernel itself; "
                                "M > 16: GEMM, then a push kernel (peer stores + flags) and a collect kernel "
                                "(b200q_gather_push)"},
            "results": results}


def _teardown_guard(seconds: float = 60.0):
    """The line has been printed; if tearing the communicator down blocks (seen once with graphs that
    had captured collectives), leave after `seconds` so that the launcher does not hang."""
    import threading

    t = threading.Timer(seconds, lambda: os._exit(0))
    t.daemon = True
    t.start()


def run_stack(args) -> None:
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    res = measure_stack(world, rank, dev, args.steps, args.warmup, tagged_rows=args.tagged_rows,
                        batches=tuple(int(b) for b in args.stack_batches.split(",")))
    if rank == 0:
        print(json.dumps({"metric": "Llama-3-8B-shaped decode linear stack, N-sharded, all-gather per layer",
                          "n_gpus": world, "steps": args.steps, "dtype": "f16", "data": "synthetic", **res}),
              flush=True)
    if world > 1:
        _teardown_guard()
        dist.barrier()
        dist.destroy_process_group()


def run_b200(args) -> None:
    import torch.distributed as dist

    from tilus_b200 import dtypes, synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = _peaks()
    dt = dtypes.uint4b
    layers = _make_layers(dt, N, K, GROUP, R_LAYERS, dev, seed=1000 * rank)
    acts = _acts(M, K, R_LAYERS, dev, seed=rank)
    graph, outs = _capture(layers, acts, ROUNDS)
    nbytes = synth.gemm_bytes(M, N, K, NBITS, GROUP)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        graph.replay()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # a step = `inner` graph replays, long enough for a few clock samples over the timed region
    inner = max(1, int(0.5 / (R_LAYERS * ROUNDS * 8e-6 * args.steps)))
    barrier()
    torch.cuda.profiler.start()  # no-op unless a profiler is attached (ncu --profile-from-start off)
    ms = _time_graph(graph, args.steps * inner)
    torch.cuda.profiler.stop()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    launches = args.steps * inner * R_LAYERS * ROUNDS
    per_launch_s = ms * 1e-3 / launches
    value = world * nbytes / per_launch_s / 1e9

    # ---- end to end through the public module, host buffers in and out --------------
    # every step copies each layer's activations from pinned host memory, runs the layer and
    # copies its result back (QuantizedLinear.forward_host); one synchronisation per step (the
    # result is read on the host)
    host_in = [a.cpu().pin_memory() for a in acts]
    host_out = [torch.empty(M, N, dtype=torch.float16).pin_memory() for _ in range(R_LAYERS)]

    def e2e_step():
        for layer, h, o in zip(layers, host_in, host_out):
            layer.forward_host(h, o)  # copy in, GEMM, copy out: one C-ABI call (b200q_gemm_host)
        torch.cuda.current_stream().synchronize()
        return float(host_out[-1][0, 0])

    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    e2e_steps = max(args.steps, 5) * 20
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / (e2e_steps * R_LAYERS)
    t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_val = world * nbytes / float(t.item()) / 1e9

    hbm = peaks["hbm_gbs"]

    def build_line(stack, cpu_baseline, extra, sweep_clocks, parity, headline_shapes):
        achieved = nbytes / per_launch_s / 1e9
        traffic = _decode_dram_traffic()
        return {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "layers_per_pass": R_LAYERS, "passes_per_graph": ROUNDS,
                       "replays_per_step": inner,
                       "l2": f"inputs larger than L2: {R_LAYERS} distinct weight sets, "
                             f"{R_LAYERS * K * N // 2 // 2**20} MiB, rotated",
                       "sharding": "replicas: one GEMV of this shape per GPU, no data-path collective "
                                   "(the sharded workload with its all-gather is `stack`)",
                       "sweep_weights": "every layer of a sweep shape holds its own copy of one synthetic weight"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s",
                         "frac": achieved / hbm,
                         "traffic": traffic["dram_bytes_per_launch"] if traffic else None,
                         "traffic_capture": {k: traffic[k] for k in ("commit", "command")} if traffic else None,
                         "peak_source": peaks["source"], "kernel": "stream_kernel<u4 zp8, MT=1>",
                         "bytes_per_launch": nbytes, "us_per_launch": per_launch_s * 1e6},
            "cpu_baseline": cpu_baseline,
            "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": R_LAYERS * M * K * 2,
                    "d2h_bytes_per_step": R_LAYERS * M * N * 2, "us_per_call": e2e_s * 1e6},
            "gpu_launches": launches,
            "clocks": clocks,
            "sweep_clocks": sweep_clocks,
            "parity": parity,
            "headline_shapes": headline_shapes,
            "stack": stack,
            "extra": extra,
        }

    prob0_a = acts[0].cpu()
    out0 = outs[0].float().cpu().numpy()
    host0 = host_out[0].float().numpy()  # what the end-to-end path left in host memory for the same layer
    del graph, layers, acts, outs
    torch.cuda.empty_cache()

    # ---- the N-sharded decode stack (strong scaling over the ranks of this run) -----------
    stack = None
    if not args.no_stack:
        import threading

        def bail():  # a rank stuck in the stack's collectives must not keep the headline number from being reported
            if rank == 0:
                print(json.dumps(build_line({"error": "no result within 300 s"}, None, {}, None, None, None)), flush=True)
            os._exit(0)

        watchdog = threading.Timer(300.0, bail)
        watchdog.daemon = True
        watchdog.start()
        try:
            stack = measure_stack(world, rank, dev, max(3, min(args.steps, 10)), args.warmup,
                                  tagged_rows=args.tagged_rows)
        except Exception as exc:  # the headline line must still be printed
            stack = {"error": f"{type(exc).__name__}: {exc}"}
        finally:
            watchdog.cancel()
        torch.cuda.empty_cache()

    if rank != 0:
        if world > 1:
            _teardown_guard()
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- correctness of what was timed ---------------------------------------------
    from oracle import quant_oracle as qo

    prob0 = synth.make_problem(1, N, K, dt, GROUP, seed=0)
    ref = qo.quantized_matmul(prob0_a.numpy(), prob0["codes"].numpy(), prob0["scales"].numpy(), dt, GROUP, 8)
    rel = float(abs(out0 - ref.astype("float32")).max() / abs(ref.astype("float32")).max())
    rel_e2e = float(abs(host0 - ref.astype("float32")).max() / abs(ref.astype("float32")).max())

    # ---- CPU baseline (bounded sample) -----------------------------------------------
    prob0["a"] = prob0_a
    cpu_s = _cpu_gemv_seconds(prob0, 5)
    cpu_baseline = {"value": nbytes / cpu_s / 1e9, "unit": "GB/s", "cores": os.cpu_count() or 1, "kind": "port",
                    "sample": "5 full M=1 K=N=8192 u4 g128 dequantize+matmul calls (oracle, torch CPU threads)"}

    # ---- extra sweep -------------------------------------------------------------------
    extra = {}
    sweep_clocks = None
    headline_shapes = {"M1_K8192_N8192_u4": {"us": round(per_launch_s * 1e6, 3), "gbs": round(nbytes / per_launch_s / 1e9, 1),
                                             "hbm_frac": round(nbytes / per_launch_s / 1e9 / hbm, 4), "rel_err": rel}}
    if world == 1 and not args.no_sweep:
        sweep_sampler = ClockSampler(local_rank)
        sweep_sampler.start()

        def mem_entry(r):
            return {"us": round(r["us"], 3), "gbs": round(r["gbs"], 1), "hbm_frac": round(r["gbs"] / hbm, 4),
                    "rel_err": float(f"{r['rel_err']:.3g}")}

        for d in (dtypes.uint1b, dtypes.uint2b, dtypes.uint3b, dtypes.uint6b, dtypes.uint8):
            extra[f"decode_{d.short_name}_M1"] = mem_entry(_sweep_shape(d, N, K, GROUP, [1], dev, 10)[1])
        r = _sweep_shape(dtypes.uint4b, 8192, 8192, GROUP, [8, 16, 32, 64], dev, 10)
        for m in (8, 16, 32, 64):
            extra[f"decode_u4_M{m}"] = mem_entry(r[m])
        headline_shapes["M16_K8192_N8192_u4"] = extra["decode_u4_M16"]
        extra["config0_u4_M16_K4096_N4096"] = mem_entry(_sweep_shape(dtypes.uint4b, 4096, 4096, GROUP, [16], dev, 10)[16])
        for d in (dtypes.float6_e3m2, dtypes.int3b):
            r = _sweep_shape(d, 4096, 4096, 4096, [1, 4, 16, 64, 256], dev, 10, scale_range=(0.5, 2.0))
            for m, v in r.items():
                extra[f"perchannel_{d.short_name}_M{m}_K4096_N4096"] = mem_entry(v)
        for name, k_in, n_out in (("qkv", 4096, 6144), ("o", 4096, 4096), ("gate_up", 4096, 28672),
                                  ("down", 14336, 4096)):
            r = _sweep_shape(dtypes.uint4b, n_out, k_in, GROUP, [1, 8, 32, 64], dev, 10)
            for m, v in r.items():
                extra[f"llama8b_{name}_M{m}"] = mem_entry(v)
        # the reference example's own table (examples/quantization/matmul_a16wx.py:551-622):
        # K=4096, N=12288, group 128, eight weight types, M in {1, 16, 4096, 4097}
        for d in (dtypes.float8_e5m2, dtypes.float6_e3m2, dtypes.float4_e2m1, dtypes.float3_e1m1, dtypes.int8,
                  dtypes.int6b, dtypes.int4b, dtypes.int3b):
            ms_list = [1, 16] if args.no_prefill else [1, 16, 4096, 4097]
            r = _sweep_shape(d, 12288, 4096, GROUP, ms_list, dev, 5)
            extra[f"example_table_{d.short_name}_K4096_N12288"] = {
                f"M{m}": {"us": round(v["us"], 2), "tflops": round(v["tflops"], 2), "gbs": round(v["gbs"], 1),
                          "rel_err": float(f"{v['rel_err']:.3g}")}
                for m, v in r.items()}
        extra.update(_sweep_followers(dev, hbm))
        if not args.no_prefill:
            r = _sweep_shape(dtypes.int4b, 28672, 8192, GROUP, [4096], dev, 3)[4096]
            extra["prefill_i4_M4096_K8192_N28672"] = {
                "ms": round(r["us"] / 1e3, 4), "tflops": round(r["tflops"], 1),
                "tensor_frac_of_measured_burst": round(r["tflops"] / peaks["tflops"], 4) if peaks["tflops"] else None,
                "tensor_frac_of_measured_sustained":
                    round(r["tflops"] / peaks["tflops_sustained"], 4) if peaks["tflops_sustained"] else None,
                "rel_err": float(f"{r['rel_err']:.3g}")}
            headline_shapes["M4096_K8192_N28672_i4"] = extra["prefill_i4_M4096_K8192_N28672"]
        sweep_clocks = sweep_sampler.stop()

    line = build_line(stack, cpu_baseline, extra, sweep_clocks,
                      {"rel_err_vs_oracle": rel, "e2e_rel_err_vs_oracle": rel_e2e, "tolerance": 1e-2}, headline_shapes)
    print(json.dumps(line), flush=True)
    if world > 1:
        _teardown_guard()
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-sweep", action="store_true", help="skip the extra dtype / shape sweep")
    ap.add_argument("--no-prefill", action="store_true", help="skip the M=4096 prefill entry of the sweep")
    ap.add_argument("--stack", action="store_true",
                    help="time the N-sharded Llama-3-8B-shaped decode linear stack (all-gather per layer) instead")
    ap.add_argument("--no-stack", action="store_true", help="skip the N-sharded decode stack")
    ap.add_argument("--stack-batches", default="1,8,32,64", help="--stack: batch sizes to run")
    ap.add_argument("--tagged-rows", type=int, default=16,
                    help="stack: batches of up to this many rows hand their rows over as tagged words (0: flags only)")
    ap.add_argument("--profile-case", default=None, choices=["decode", "batch16", "batch32", "prefill"],
                    help="run a few plain launches of one kernel (for ncu) instead of the benchmark")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.profile_case:
        run_profile_case(args)
    elif args.stack:
        run_stack(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
