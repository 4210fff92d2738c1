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

import ctypes

from . import _lib, ops, packing
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
                 process_group=None, gather_output: bool = True, shard=None):
        super().__init__()
        self.process_group = process_group
        if shard is not None:  # explicit (world, rank): shards handled by one process, e.g. in tests
            self.world, self.rank = shard
        else:
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
        if self.gather_output and self.world > 1 and dist.is_initialized():
            y = gather_columns(y, self.process_group)
        return y


# ---------------------------------------------------------------------------------------------
# fused all-gather: the GEMV kernel stores its columns straight into every rank's output row
# ---------------------------------------------------------------------------------------------
class _RawCudaBuffer:
    """A device pointer as an object torch.as_tensor understands (CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class GatheredRow:
    """The gathered output of the latest fused call of a PeerGather context, or a column range of
    it, as the activations of the next call.  Which of the two row buffers holds it is only known
    on the device; PeerGather.fetch brings it to a tensor."""

    def __init__(self, rows: int, row_stride: int, col_start: int, width: int, tagged: bool = False):
        self.rows, self.row_stride, self.col_start, self.width = rows, row_stride, col_start, width
        self.tagged = tagged  # which of the context's two hand-over protocols produced it

    def cols(self, start: int, stop: int) -> "GatheredRow":
        assert 0 <= start < stop <= self.width and start % 8 == 0
        return GatheredRow(self.rows, self.row_stride, self.col_start + start, stop - start, self.tagged)


class PeerGather:
    """Peer-mapped output rows and arrival flags for the fused all-gather of a column-sharded
    decode stack (include/b200q.h, b200q_gemm_gather).

    Every rank owns one region: `world` 32-bit flags, a call counter, and two fp16 row buffers
    [max_rows, max_cols] used alternately.  `ptrs[g]` is rank g's region as seen from this
    process.  A fused call waits (on the device) until every rank has finished the previous
    call, writes its columns into the other row buffer of every rank and raises its flag on
    every rank; the call counter lives on the device, so the calls carry no per-call state and
    a sequence of them can be captured in a CUDA graph and replayed.  All ranks must make the
    same sequence of calls.

    Batches of at most `tagged_rows` rows (default 16: every fused call) use the tagged hand-over instead
    (B200Q_GATHER_TAGGED): three more row buffers of 8-byte words {two outputs, call number} and a call
    counter of their own; no flags, no grid-wide wait - the next call (or, above 16 rows, the collect
    kernel) polls the words it reads.  Above 16 rows the flags are faster (twice the bytes to push and to
    poll: 3.11 vs 2.91 ms at M = 32 on two GPUs), so the default leaves those batches on flags.
    Measured on two B200s over NVLink (128-linear decode stack): 1.71 -> 1.51 ms per step at M = 1,
    1.80 -> 1.66 ms at M = 8.
    """

    FLAGS_OFF, EPOCH_OFF, TAG_EPOCH_OFF, ROWS_OFF = 0, 64, 128, 256
    TAG_BUFFERS = 3

    def __init__(self, world: int, rank: int, ptrs, max_rows: int, max_cols: int, device, tagged_rows: int = 16):
        assert 1 <= world <= 8 and len(ptrs) == world
        self.world, self.rank, self.ptrs = world, rank, list(ptrs)
        self.max_rows, self.max_cols = max_rows, max_cols
        self.tagged_rows = min(tagged_rows, max_rows)
        self._tag_prev = None  # (rows, row width, took its activations from outside) of the latest tagged call
        self.device = torch.device(device)
        self._owned = None     # this rank's region, if allocated by create()
        self._full = {}        # gathered outputs of calls with more than 16 rows, per shape
        self._opened = []      # peers' regions mapped by create()
        self.dtype = torch.float16  # dtype of the latest call's output rows

    @staticmethod
    def _tag_off(max_rows: int, max_cols: int) -> int:
        return (PeerGather.ROWS_OFF + 2 * max_rows * max_cols * 2 + 255) // 256 * 256

    @staticmethod
    def region_bytes(max_rows: int, max_cols: int, tagged_rows: int = 16) -> int:
        tagged_rows = min(tagged_rows, max_rows)
        return PeerGather._tag_off(max_rows, max_cols) + PeerGather.TAG_BUFFERS * tagged_rows * (max_cols // 2) * 8

    @classmethod
    def create(cls, max_rows: int, max_cols: int, device, group=None, tagged_rows: int = 16):
        """Allocates this rank's region with the library's peer allocator (zeroed) and maps every
        other rank's region through CUDA IPC (one process per GPU, one node)."""
        lib = _lib.load()
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        nbytes = cls.region_bytes(max_rows, max_cols, tagged_rows)
        with torch.cuda.device(device):
            mine = ctypes.c_void_p()
            _lib.check(lib.b200q_peer_alloc(nbytes, ctypes.byref(mine)))
            handle = ctypes.create_string_buffer(64)
            _lib.check(lib.b200q_peer_export(mine, handle))
            handles = [None] * world
            if world > 1:
                dist.all_gather_object(handles, bytes(handle.raw), group=group)
            ptrs = []
            for g in range(world):
                if g == rank:
                    ptrs.append(mine.value)
                else:
                    peer = ctypes.c_void_p()
                    _lib.check(lib.b200q_peer_open(ctypes.create_string_buffer(handles[g], 64), ctypes.byref(peer)))
                    ptrs.append(peer.value)
        ctx = cls(world, rank, ptrs, max_rows, max_cols, device, tagged_rows)
        ctx._owned = mine.value
        ctx._opened = [p for g, p in enumerate(ptrs) if g != rank]
        ctx._group = group
        return ctx

    def close(self):
        """Unmaps the peers' regions and frees this rank's own (only what create() made).  Every rank
        must have finished its fused calls: a barrier precedes the release when a process group is up."""
        if self._owned is None:
            return
        lib = _lib.load()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            if dist.is_initialized() and self.world > 1:
                dist.barrier(group=getattr(self, "_group", None))
            for p in self._opened:
                _lib.check(lib.b200q_peer_close(ctypes.c_void_p(p)))
            _lib.check(lib.b200q_peer_free(ctypes.c_void_p(self._owned)))
        self._opened, self._owned = [], None

    def _view(self, byte_off: int, nbytes: int) -> torch.Tensor:
        return torch.as_tensor(_RawCudaBuffer(self.ptrs[self.rank] + byte_off, nbytes), device=self.device)

    def _desc(self, N_full: int, col_offset: int, tagged: bool = False) -> "_lib.Gather":
        g = _lib.Gather()
        g.world, g.rank, g.ldc, g.col_offset = self.world, self.rank, N_full, col_offset
        g.a_prev_offset = -1
        if tagged:
            off = self._tag_off(self.max_rows, self.max_cols)
            g.mode = _lib.GATHER_TAGGED
            for r in range(self.world):
                g.out[r] = self.ptrs[r] + off
            g.epoch_local = self.ptrs[self.rank] + self.TAG_EPOCH_OFF
            g.buffer_elems = self.tagged_rows * (self.max_cols // 2)
            return g
        for r in range(self.world):
            g.out[r] = self.ptrs[r] + self.ROWS_OFF
            g.flag_slot[r] = self.ptrs[r] + self.FLAGS_OFF + 4 * self.rank
        g.flags_local = self.ptrs[self.rank] + self.FLAGS_OFF
        g.epoch_local = self.ptrs[self.rank] + self.EPOCH_OFF
        g.buffer_elems = self.max_rows * self.max_cols
        g.a_prev_offset = -1
        return g

    def gemm(self, x, layer: "ShardedQuantizedLinear"):
        """One call: this rank's columns of layer(x), gathered into every rank's row buffer.  x is a
        tensor [M, K] or what the previous call returned (or a column range of it, `cols`).

        Up to 16 rows the GEMV kernel itself stores into every rank's buffer (b200q_gemm_gather) and the
        result is a GatheredRow - a handle whose buffer only the device knows; the next call takes it
        as its activations, `fetch` brings it to a tensor.  Above 16 rows the local GEMM runs as usual
        and two small kernels push its shard to every rank and collect the complete rows
        (b200q_gather_push); the result is an ordinary tensor [M, N] owned by this context (valid
        until the next call with the same shape)."""
        lib = _lib.load()
        local = layer.local
        N_full, N_loc, K = layer.out_features, local.out_features, layer.in_features
        dt, zp, grp = local.w_dtype, local.zero_point, local.group_size
        if isinstance(x, GatheredRow):
            M = x.rows
        else:
            if x.dtype != local.scales.dtype or x.stride(1) != 1 or x.shape[1] != K:
                raise TypeError(f"activations must be {local.scales.dtype} [M, {K}] with unit inner stride")
            M = x.shape[0]
        if M > self.max_rows or N_full > self.max_cols:
            raise ValueError("batch or layer width beyond the context's buffer size")
        tagged = M <= self.tagged_rows and self.world > 1  # a single rank has no hand-over to shorten
        g = self._desc(N_full, layer.n0, tagged)
        self.dtype = local.scales.dtype
        if M > 16:
            if isinstance(x, GatheredRow):
                raise ValueError("a GatheredRow feeds fused calls (M <= 16) only")
            with torch.cuda.device(self.device):
                shard = local(x)
                full = self._full.get((M, N_full, self.dtype))
                if full is None:
                    full = torch.empty(M, N_full, dtype=self.dtype, device=self.device)
                    self._full[(M, N_full, self.dtype)] = full
                self.push(shard, layer, tagged)
                self.collect(full, M, N_full, tagged)
            if tagged:
                self._tag_prev = (M, N_full, False)  # collected: nothing of it is left to wait for
            return full
        if isinstance(x, GatheredRow):
            lda, a_ptr = x.row_stride, None
            if x.width != K:
                raise ValueError(f"expected {K} input features, got {x.width}")
            if x.tagged != tagged:
                raise ValueError("the previous call's rows were handed over with the other protocol")
            g.a_prev_offset = x.col_start
        else:
            lda, a_ptr = x.stride(0), x.data_ptr()
            if tagged and self._tag_prev is not None and self._tag_prev[2]:
                # two tagged calls in a row that take their activations from outside: make sure every rank
                # has written the first one's rows (so it has finished reading the buffer written next)
                self.collect(None, self._tag_prev[0], self._tag_prev[1], tagged=True)
        if tagged:
            self._tag_prev = (M, N_full, not isinstance(x, GatheredRow))
        with torch.cuda.device(self.device):
            ws = ops.get_workspace(self.device, ops.workspace_bytes(M, N_loc, K, dt, zp, grp))
            st = lib.b200q_gemm_gather(a_ptr, lda, local.quantized_weight.data_ptr(), local.scales.data_ptr(), M,
                                       N_loc, K, dt.code, zp, grp, ops.act_code(local.scales.dtype), ws.data_ptr(),
                                       ws.numel(),
                                       torch.cuda.current_stream(self.device).cuda_stream, ctypes.byref(g))
        _lib.check(st)
        return GatheredRow(M, N_full, 0, N_full, tagged)

    def push(self, shard: torch.Tensor, layer: "ShardedQuantizedLinear", tagged: bool = False):
        """First half of a gathered call with more than 16 rows: this rank's shard [M, N/G] to every rank
        (dense rows + flags, or tagged words)."""
        g = self._desc(layer.out_features, layer.n0, tagged)
        with torch.cuda.device(self.device):
            ws = ops.get_workspace(self.device, 1 << 20)
            _lib.check(_lib.load().b200q_gather_push(
                shard.data_ptr(), shard.stride(0), shard.shape[0], shard.shape[1], ws.data_ptr(), ws.numel(),
                torch.cuda.current_stream(self.device).cuda_stream, ctypes.byref(g)))

    def collect(self, full, M: int, N_full: int, tagged: bool = False):
        """Second half: wait for every rank's shard of the call just pushed (or, tagged, of the latest
        fused call), copy the rows to `full` (None: wait only)."""
        g = self._desc(N_full, 0, tagged)
        with torch.cuda.device(self.device):
            ws = ops.get_workspace(self.device, 1 << 20)
            _lib.check(_lib.load().b200q_gather_collect(
                full.data_ptr() if full is not None else None, full.stride(0) if full is not None else 0, M,
                ws.data_ptr(), ws.numel(), torch.cuda.current_stream(self.device).cuda_stream, ctypes.byref(g)))

    @staticmethod
    def cols(row, start: int, stop: int):
        """Columns [start, stop) of what `gemm` returned, as the activations of the next call."""
        return row.cols(start, stop) if isinstance(row, GatheredRow) else row[:, start:stop]

    def calls_completed(self, tagged: bool = False) -> int:
        """The device-side call counter of the flag protocol (or of the tagged one); synchronises the
        current stream."""
        torch.cuda.current_stream(self.device).synchronize()
        return int(self._view(self.TAG_EPOCH_OFF if tagged else self.EPOCH_OFF, 4).view(torch.int32).item())

    def wait_all_ranks(self, timeout_s: float = 2.0) -> int:
        """Waits until every rank's columns of this rank's latest call have landed here: this rank's
        own stream is synchronised, then its flag words - one per source rank, raised over NVLink by
        that rank's kernel - are polled until all have reached the call counter (bounded)."""
        import time

        epoch = self.calls_completed()
        flags = self._view(self.FLAGS_OFF, 4 * self.world).view(torch.int32)
        t0 = time.perf_counter()
        while True:
            seen = flags.cpu()
            if bool(((seen - epoch) >= 0).all()):
                return epoch
            if time.perf_counter() - t0 > timeout_s:
                raise _lib.B200QError(_lib.ST_DEVICE_TIMEOUT, f"fused gather: flags {seen.tolist()} never reached call {epoch}")
            time.sleep(0.0005)

    def fetch(self, row) -> torch.Tensor:
        """The latest call's gathered output (or the column range `row` of it) as a new tensor, once
        every rank's columns are in place."""
        if not isinstance(row, GatheredRow):  # more than 16 rows: already collected on the device
            torch.cuda.current_stream(self.device).synchronize()
            return row.clone()
        if row.tagged:  # the collect kernel waits for every word's tag and writes dense rows
            full = torch.empty(row.rows, row.row_stride, dtype=self.dtype, device=self.device)
            self.collect(full, row.rows, row.row_stride, tagged=True)
            torch.cuda.current_stream(self.device).synchronize()
            st = ops.device_status(ops.get_workspace(self.device, 1 << 20))
            if st[0] != 0:
                raise _lib.B200QError(_lib.ST_DEVICE_TIMEOUT, f"tagged gather: rows never completed, status {st}")
            return full[:, row.col_start : row.col_start + row.width].clone()
        parity = self.wait_all_ranks() & 1
        nbytes = self.max_rows * self.max_cols * 2
        buf = self._view(self.ROWS_OFF + parity * nbytes, nbytes).view(self.dtype)
        full = buf[: row.rows * row.row_stride].view(row.rows, row.row_stride)
        return full[:, row.col_start : row.col_start + row.width].clone()
