"""Column sharding and the output all-gather, world size 2, gloo on CPU.

The per-rank matmul needs a GPU, so here each rank's local output is produced by the oracle
from the codes recovered from its own shard of the packed weights; what is under test is the
host logic: shard ranges, the contiguous-byte-range property of the packed layout, and the
gather into the full row for M == 1 and M > 1."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, M, result_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import quant_oracle as qo
        from tilus_b200 import dtypes as D
        from tilus_b200 import packing, sharded, synth

        K, N, g = 512, 128, 128
        dt = D.int4b
        prob = synth.make_problem(M, N, K, dt, g, seed=7)
        full = packing.interleave(prob["codes"], dt)
        n0, n1 = sharded.shard_range(N, world, rank)
        assert (n1 - n0) * world == N and n0 % 16 == 0
        part = packing.shard_columns(full, dt, K, N, n0, n1)
        # the shard of the full packed matrix is the packed shard
        assert torch.equal(part, packing.interleave(prob["codes"][:, n0:n1].contiguous(), dt))
        codes_local = packing.deinterleave(part.clone(), dt, K, n1 - n0).numpy()
        local = qo.quantized_matmul(prob["a"].numpy(), codes_local, prob["scales"][:, n0:n1].numpy(), dt, g, 0)
        got = sharded.gather_columns(torch.from_numpy(local))
        want = qo.quantized_matmul(prob["a"].numpy(), prob["codes"].numpy(), prob["scales"].numpy(), dt, g, 0)
        assert got.shape == (M, N)
        np.testing.assert_array_equal(got.numpy().view(np.uint16), want.view(np.uint16))
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("M", [1, 5])
def test_shard_and_gather_world2(tmp_path, M):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), M, str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(tmp_path / f"ok{r}") for r in range(world))


def test_shard_range_rules():
    sys.path.insert(0, ROOT)
    from tilus_b200 import sharded

    assert sharded.shard_range(6144, 8, 3) == (2304, 3072)
    assert sharded.shard_range(28672, 8, 7) == (25088, 28672)
    with pytest.raises(ValueError):
        sharded.shard_range(4096 + 16, 8, 0)
