"""Column-sharded (N-sharded) quantized linear layers for one node of several GPUs.

The weight-only quantized matmul shards naturally by output columns: rank r of G holds
Bq[:, n0:n1] (a contiguous byte range of the packed weights, packing.shard_columns),
scales[:, n0:n1] and the replicated activations, and computes C[:, n0:n1].  The only
exchange is an all-gather of the [M, N/G] fp16 outputs, and only where the next operator
needs the full row.  The reference is single-GPU (no collective anywhere in its tree), so
this module has no counterpart there; the per-rank operator is QuantizedLinear
(examples/quantization/matmul_a16wx.py:408-548 of the reference).

One process per GPU, torch.distributed for the plumbing (NCCL over NVLink on GPUs; the
range / gather logic is backend-agnostic and is exercised on CPU with gloo).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

from . import packing
from .dtypes import weight_dtype
from .linear import QuantizedLinear

SHARD_MULTIPLE = packing.BLOCK_N  # column shards are whole 16-column tiles


def shard_range(n: int, world: int, rank: int, multiple: int = SHARD_MULTIPLE):
    """Columns [n0, n1) of rank `rank`: equal contiguous slices, each a multiple of `multiple`."""
    if n % (world * multiple) != 0:
        raise ValueError(f"out_features={n} cannot be split in {world} equal shards of whole {multiple}-column tiles")
    per = n // world
    return rank * per, (rank + 1) * per


def gather_columns(local: torch.Tensor, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather column shards local[M, N/G] into [M, N].  For M == 1 the gathered buffer is
    already the output row; otherwise the [G, M, N/G] buffer is permuted once."""
    world = dist.get_world_size(group)
    if world == 1:
        return local
    M, nl = local.shape
    buf = torch.empty(world * M, nl, dtype=local.dtype, device=local.device)  # [G][M][N/G]
    dist.all_gather_into_tensor(buf, local.contiguous(), group=group)
    if M == 1:
        res = buf.view(1, world * nl)
    else:
        res = buf.view(world, M, nl).permute(1, 0, 2).reshape(M, world * nl)
    if out is not None:
        out.copy_(res)
        return out
    return res


class ShardedQuantizedLinear(nn.Module):
    """QuantizedLinear whose out_features are split over the ranks of a process group."""

    def __init__(self, x_dtype, w_dtype, group_size: int, in_features: int, out_features: int, zero_point: int = 0,
                 process_group=None, gather_output: bool = True):
        super().__init__()
        self.process_group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        self.in_features, self.out_features = in_features, out_features
        self.n0, self.n1 = shard_range(out_features, self.world, self.rank)
        self.gather_output = gather_output
        self.w_dtype = weight_dtype(w_dtype)
        self.local = QuantizedLinear(x_dtype, w_dtype, group_size, in_features, self.n1 - self.n0, zero_point=zero_point)

    def load_codes(self, codes: torch.Tensor, scales: torch.Tensor):
        """Full codes uint8[K, N] and scales [K/g, N]; every rank keeps its own columns."""
        self.local.load_codes(codes[:, self.n0:self.n1].contiguous(), scales[:, self.n0:self.n1].contiguous())

    def load_packed_full(self, storage: torch.Tensor, scales: torch.Tensor):
        """Full b200-packed weights: the shard is a contiguous byte range."""
        part = packing.shard_columns(storage, self.w_dtype, self.in_features, self.out_features, self.n0, self.n1)
        self.local.load_packed(part, scales[:, self.n0:self.n1].contiguous(), layout="b200")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.local(x)
        if self.gather_output and self.world > 1:
            y = gather_columns(y, self.process_group)
        return y
