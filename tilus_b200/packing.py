"""Host-side weight re-packer (PyTorch).

Three byte formats of a b-bit weight matrix q[K, N] appear here; all have exactly
K*N*b/8 bytes:

``canonical``  the reference's ``tilus.Tensor`` storage: row-major, bit-dense,
               little-endian; element i = k*N + n occupies bits [i*b, (i+1)*b)
               (python/tilus/tensor.py:112-115,
               python/tilus/hidet/ir/primitives/cuda/subbyte.py:36-52).
``ref_tiled``  what the reference's QuantizedLinear keeps in ``quantized_weight``:
               uint8[K/16, N/16, 32*b] in mma.sync B-fragment order
               (examples/quantization/matmul_a16wx.py:64-98).
``b200``       this library's private interleave, consumed by the sm_100a kernels
               (layout version LAYOUT_VERSION), described below.

The b200 layout
---------------
*Unit*: the 32 codes q[k0 .. k0+31, n] of one column n (k0 % 32 == 0) are stored in
b consecutive 32-bit words.  b is split into bit planes of width 8/4/2/1, most
significant first (``PLANES``): 3 = 2+1, 5 = 4+1, 6 = 4+2, 7 = 4+2+1.  A plane of
width p takes p words; pair h = 0..15 (codes k0+2h and k0+2h+1) sits in plane word
h // (16/p) as field f = h % (16/p): the even-k field in bits [f*p, f*p+p) and the
odd-k field in bits [16+f*p, 16+f*p+p).  One mask therefore isolates a k-adjacent
pair as the two 16-bit halves of a register, ready for the fp16 magic-number
conversion.  Signed integer codes are stored with the sign bit flipped (offset
binary) so that signed and unsigned types decode with one subtraction.

*Group*: 16 columns x 128 rows = 16 columns x 4 units of 32.  Inside group g of column tile nt
the units are ordered [half = 0..1][lane = 0..31] with lane = r*4 + j holding column
n = nt*16 + half*8 + r, rows g*128 + j*32 + [0, 32), each unit as its b words: word offset
(half*32 + lane)*b + v.  So a 128-row group (one scale per column when group_size is a
multiple of 128) is 256*b contiguous bytes, the four lanes that share a column split a group
in 32-row units, and the 128 rows of one column of a group are 16*b contiguous bytes.  Four
consecutive groups form a 512-row *block* of 1024*b contiguous bytes, the unit of work of the
decode kernel.

*Matrix*: groups in [nt][g] order (column-tile major, g = 0 .. K/128 - 1), so a contiguous
range of column tiles - an N shard - is a contiguous byte range.  K must be a multiple of
128 (the decode kernel for up to 16 rows wants whole blocks, K a multiple of 512; other K
run on the tensor-core kernels).
"""
from __future__ import annotations

import torch

from .dtypes import KIND_INT, WeightDType, weight_dtype

LAYOUT_VERSION = 1
BLOCK_N = 16
BLOCK_K = 512
GROUP_K = 128
UNIT_K = 32

PLANES = {1: (1,), 2: (2,), 3: (2, 1), 4: (4,), 5: (4, 1), 6: (4, 2), 7: (4, 2, 1), 8: (8,)}


# ---------------------------------------------------------------------------
# canonical <-> codes
# ---------------------------------------------------------------------------
def unpack_canonical(storage: torch.Tensor, nbits: int, K: int, N: int) -> torch.Tensor:
    """canonical bytes -> codes uint8[K, N]."""
    st = storage.reshape(-1).to(torch.uint8)
    assert st.numel() * 8 == K * N * nbits, "storage size mismatch"
    if nbits == 8:
        return st.reshape(K, N).clone()
    shifts = torch.arange(8, dtype=torch.uint8, device=st.device)
    bits = (st[:, None] >> shifts) & 1  # little-endian bit stream
    bits = bits.reshape(K * N, nbits)
    weights = (1 << torch.arange(nbits, device=st.device)).to(torch.uint8)
    return (bits * weights).sum(dim=1, dtype=torch.int32).to(torch.uint8).reshape(K, N)


def pack_canonical(codes: torch.Tensor, nbits: int) -> torch.Tensor:
    """codes uint8[K, N] -> canonical bytes."""
    flat = codes.reshape(-1).to(torch.uint8)
    assert (flat.numel() * nbits) % 8 == 0
    if nbits == 8:
        return flat.clone()
    shifts = torch.arange(nbits, dtype=torch.uint8, device=flat.device)
    bits = ((flat[:, None] >> shifts) & 1).reshape(-1, 8)
    weights = (1 << torch.arange(8, device=flat.device)).to(torch.int32)
    return (bits.to(torch.int32) * weights).sum(dim=1).to(torch.uint8)


def _ref_tile_bit_map(nbits: int) -> torch.Tensor:
    """[16*16*b] absolute bit index inside a 32*b-byte reference tile, ordered
    (k, n, bit).  Lane/slot rule of examples/quantization/matmul_a16wx.py:29-61."""
    from math import gcd

    k = torch.arange(16)[:, None, None]
    n = torch.arange(16)[None, :, None]
    bit = torch.arange(nbits)[None, None, :]
    lane = (n % 8) * 4 + (k % 8) // 2
    slot = (n // 8) * 4 + (k // 8) * 2 + (k % 2)
    inner = gcd(nbits, 16)
    lane_bit = slot * nbits + bit
    j = lane_bit // 8
    o, i = j // inner, j % inner
    return ((o * 32 * inner + lane * inner + i) * 8 + lane_bit % 8).reshape(-1)


def unpack_ref_tiled(storage: torch.Tensor, nbits: int, K: int, N: int) -> torch.Tensor:
    """The reference's ``quantized_weight`` bytes -> codes uint8[K, N]."""
    st = storage.reshape(-1).to(torch.uint8)
    assert st.numel() * 8 == K * N * nbits, "storage size mismatch"
    shifts = torch.arange(8, dtype=torch.uint8, device=st.device)
    bits = ((st[:, None] >> shifts) & 1).reshape(K // 16, N // 16, 32 * nbits * 8)
    bmap = _ref_tile_bit_map(nbits).to(st.device)
    src = bits[:, :, bmap].reshape(K // 16, N // 16, 16, 16, nbits).to(torch.int32)
    weights = (1 << torch.arange(nbits, device=st.device)).to(torch.int32)
    tiles = (src * weights).sum(dim=-1).to(torch.uint8)
    return tiles.permute(0, 2, 1, 3).reshape(K, N).contiguous()


def pack_ref_tiled(codes: torch.Tensor, nbits: int) -> torch.Tensor:
    """codes uint8[K, N] -> the reference's ``quantized_weight`` bytes."""
    K, N = codes.shape
    tiles = codes.reshape(K // 16, 16, N // 16, 16).permute(0, 2, 1, 3).to(torch.uint8)
    shifts = torch.arange(nbits, dtype=torch.uint8, device=codes.device)
    src_bits = ((tiles[..., None] >> shifts) & 1).reshape(K // 16, N // 16, -1)
    out_bits = torch.zeros(K // 16, N // 16, 32 * nbits * 8, dtype=torch.uint8, device=codes.device)
    out_bits[:, :, _ref_tile_bit_map(nbits).to(codes.device)] = src_bits
    weights = (1 << torch.arange(8, device=codes.device)).to(torch.int32)
    return (out_bits.reshape(-1, 8).to(torch.int32) * weights).sum(dim=1).to(torch.uint8)


# ---------------------------------------------------------------------------
# codes <-> b200 interleave
# ---------------------------------------------------------------------------
def check_shape(K: int, N: int) -> None:
    if K % GROUP_K != 0 or N % BLOCK_N != 0:
        raise ValueError(
            f"b200 weight layout needs in_features % {GROUP_K} == 0 and out_features % {BLOCK_N} == 0, "
            f"got K={K}, N={N}"
        )


def stored_codes(codes: torch.Tensor, dt: WeightDType) -> torch.Tensor:
    """Codes as kept in the b200 layout: signed integers in offset binary."""
    if dt.kind == KIND_INT:
        return codes ^ (1 << (dt.nbits - 1))
    return codes


def _unit_words(codes: torch.Tensor, nbits: int) -> torch.Tensor:
    """codes int32[..., 32] (one unit along the last axis) -> words int32[..., b]."""
    lead = codes.shape[:-1]
    c = codes.reshape(*lead, 16, 2).to(torch.int64)  # [.., h, e]
    words = []
    lo = nbits
    for p in PLANES[nbits]:
        lo -= p
        field = (c >> lo) & ((1 << p) - 1)  # [.., 16, 2]
        per_word = 16 // p
        field = field.reshape(*lead, p, per_word, 2)  # [.., word, f, e]
        f = torch.arange(per_word, device=codes.device).reshape(per_word, 1)
        e = torch.arange(2, device=codes.device).reshape(1, 2)
        sh = f * p + 16 * e
        w = (field << sh).sum(dim=(-1, -2))  # [.., word]
        words.append(w)
    out = torch.cat(words, dim=-1)  # [.., b]
    out = torch.where(out >= (1 << 31), out - (1 << 32), out)
    return out.to(torch.int32)


def _words_to_codes(words: torch.Tensor, nbits: int) -> torch.Tensor:
    """Inverse of _unit_words: words int32[..., b] -> codes uint8[..., 32]."""
    lead = words.shape[:-1]
    w = words.to(torch.int64) & 0xFFFFFFFF
    codes = torch.zeros(*lead, 16, 2, dtype=torch.int64, device=words.device)
    lo = nbits
    base = 0
    for p in PLANES[nbits]:
        lo -= p
        per_word = 16 // p
        pw = w[..., base : base + p]  # [.., word]
        f = torch.arange(per_word, device=words.device).reshape(per_word, 1)
        e = torch.arange(2, device=words.device).reshape(1, 2)
        sh = f * p + 16 * e
        field = (pw[..., None, None] >> sh) & ((1 << p) - 1)  # [.., word, f, e]
        codes |= field.reshape(*lead, 16, 2) << lo
        base += p
    return codes.reshape(*lead, 32).to(torch.uint8)


def interleave(codes: torch.Tensor, dt, chunk_tiles: int = 64) -> torch.Tensor:
    """codes uint8[K, N] (as decoded by the type: two's complement for intNb) ->
    b200 bytes uint8[K*N*b/8]."""
    dt = weight_dtype(dt)
    b = dt.nbits
    K, N = codes.shape
    check_shape(K, N)
    G, NT = K // GROUP_K, N // BLOCK_N
    out = torch.empty(NT, G, 2, 32, b, dtype=torch.int32, device=codes.device)
    sc = stored_codes(codes.to(torch.uint8), dt)
    for t0 in range(0, NT, chunk_tiles):
        t1 = min(NT, t0 + chunk_tiles)
        blk = sc[:, t0 * 16 : t1 * 16].reshape(G, 4, 32, t1 - t0, 2, 8)  # g j i nt half r
        blk = blk.permute(3, 0, 4, 5, 1, 2)  # nt g half r j i
        words = _unit_words(blk.to(torch.int32), b)  # nt g half r j v
        out[t0:t1] = words.reshape(t1 - t0, G, 2, 32, b)
    return out.reshape(-1).view(torch.uint8)


def deinterleave(storage: torch.Tensor, dt, K: int, N: int) -> torch.Tensor:
    """b200 bytes -> codes uint8[K, N] (inverse of interleave)."""
    dt = weight_dtype(dt)
    b = dt.nbits
    check_shape(K, N)
    G, NT = K // GROUP_K, N // BLOCK_N
    st = storage.reshape(-1).contiguous()
    assert st.dtype == torch.uint8 and st.numel() * 8 == K * N * b
    words = st.view(torch.int32).reshape(NT, G, 2, 8, 4, b)  # nt g half r j v
    codes = _words_to_codes(words, b)  # nt g half r j i
    codes = codes.permute(1, 4, 5, 0, 2, 3).reshape(K, N)  # g j i nt half r
    return stored_codes(codes.contiguous(), dt)


def shard_columns(storage: torch.Tensor, dt, K: int, N: int, n0: int, n1: int) -> torch.Tensor:
    """Bytes of columns [n0, n1) of a b200-packed matrix: a contiguous slice."""
    dt = weight_dtype(dt)
    assert n0 % BLOCK_N == 0 and n1 % BLOCK_N == 0
    per_tile = K * BLOCK_N * dt.nbits // 8
    return storage.reshape(-1)[n0 // BLOCK_N * per_tile : n1 // BLOCK_N * per_tile]
