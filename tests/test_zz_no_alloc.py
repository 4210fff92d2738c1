"""b200q_gemm_static_ws - the entry point for callers that may not allocate device memory -
against b200q_gemm on the same inputs.

Collected last on purpose (file name), so that a run which stops at the first failure has
already been through every other test.  It must pass alone in a fresh process and after the
rest of the suite: both entry points are driven here through the C ABI with explicit buffers.
"""
import ctypes

import numpy as np
import pytest
import torch

from tilus_b200 import _lib, packing, synth
from tilus_b200 import dtypes as D

pytestmark = pytest.mark.gpu

REL_TOL = 1e-2  # the tolerance of the other GEMM parity tests


def _gemm_both(M, N, K, dt, group, seed):
    lib = _lib.load()
    dev = torch.device("cuda:0")
    prob = synth.make_problem(M, N, K, dt, group, seed=seed)
    zp = prob["zero_point"]
    a = prob["a"].to(dev)
    bq = packing.interleave(prob["codes"], dt).to(dev)
    sc = prob["scales"].to(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream

    need = lib.b200q_workspace_bytes(M, N, K, dt.code, zp, group)
    assert 0 < need <= lib.b200q_static_workspace_limit()
    ws = torch.zeros(need, dtype=torch.uint8, device=dev)
    c_ref = torch.empty(M, N, dtype=torch.float16, device=dev)
    _lib.check(lib.b200q_gemm(a.data_ptr(), K, bq.data_ptr(), sc.data_ptr(), c_ref.data_ptr(), N, M, N, K, dt.code, zp,
                              group, _lib.ACT_F16, ws.data_ptr(), ws.numel(), stream))
    _lib.check(lib.b200q_static_ws_init())  # set-up time: the module with the array is loaded here
    outs = [torch.full((M, N), float("nan"), dtype=torch.float16, device=dev) for _ in range(2)]
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(dev)[0]
    for c in outs:  # the second call runs on the scratch the first one left behind
        _lib.check(lib.b200q_gemm_static_ws(a.data_ptr(), K, bq.data_ptr(), sc.data_ptr(), c.data_ptr(), N, M, N, K,
                                            dt.code, zp, group, _lib.ACT_F16, stream))
    torch.cuda.synchronize()
    # nothing was allocated by the calls: the device's free memory is what it was after set-up
    assert torch.cuda.mem_get_info(dev)[0] == free_before
    # no bounded wait gave up; the status query reads the built-in scratch (workspace = NULL)
    status = (ctypes.c_int32 * 4)()
    assert lib.b200q_device_status(None, ctypes.byref(status), stream) == _lib.ST_OK
    assert list(status) == [0, 0, 0, 0]
    return c_ref.float().cpu().numpy(), [o.float().cpu().numpy() for o in outs]


@pytest.mark.parametrize("M,N,K", [(200, 256, 2048), (40, 256, 2048), (3, 272, 2048)])
def test_static_workspace_matches_gemm_twice(M, N, K):
    # (200, 256, 2048) and (40, 256, 2048) run the two tcgen05 kernels with split-K, (3, 272, 2048) the
    # mma.sync kernel with column tiles shared between CTAs: in all of them fp32 partial sums and
    # arrival counters live in the built-in scratch
    ref, outs = _gemm_both(M, N, K, D.int4b, 128, seed=21)
    scale = np.abs(ref).max()
    for got in outs:
        assert np.isfinite(got).all()
        assert np.abs(got - ref).max() / scale <= REL_TOL


def test_static_workspace_rejects_oversize():
    """A problem whose scratch does not fit the built-in array is refused before anything is
    launched (so the placeholder buffers below are never touched)."""
    lib = _lib.load()
    limit = lib.b200q_static_workspace_limit()
    M, N, K = 8, 262144, 512  # the decode kernel's fp32 scratch is 16 * N * 4 bytes = 16 MiB
    dt = D.int4b
    need = lib.b200q_workspace_bytes(M, N, K, dt.code, 0, 128)
    assert need > limit
    dev = torch.device("cuda:0")
    dummy = torch.zeros(64, dtype=torch.uint8, device=dev)
    st = lib.b200q_gemm_static_ws(dummy.data_ptr(), K, dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), N, M, N,
                                  K, dt.code, 0, 128, _lib.ACT_F16, None)
    assert st == _lib.ST_WORKSPACE
    assert b"workspace" in lib.b200q_status_string(st)
