"""B200 execution layouts derived from the canonical artifacts (offline, once per layer).

The canonical ``xqt_int4_nk_v1`` tensors stay the serialised form; what is built here is a
backend-private cache, like xqt's ``sm89_awq_w4a16_interleaved_v1`` execution layout that keeps
``canonical_qweight`` beside it (xqt/kernels/ops/_impl/gemm_backends/sm89/awq_w4a16_decode_sm89.py:16-98,
pack kernel xqt/kernels/jit/csrc/quantization/awq_w4a16_sm89_kernel.cu:405-479).

``b200_w4_tile128_v1`` (decode GEMV):
  weights  uint8 ``[N/128 tiles][K/128 kblocks][16 ntiles][32 lanes][16 bytes]``
           One (tile, kblock) unit is 8 KiB contiguous, consecutive kblocks of a tile are adjacent,
           so a pipeline stage is ONE bulk copy.  Lane ``4*g + t`` of ntile ``j`` holds channel
           ``128*tile + 8*j + g``; its 32-bit word ``w`` holds ``k = 128*kblock + 32*w + 8*t + e``
           with ``e = 0,2,4,6,1,3,5,7`` in nibble positions 0..7, so that
           ``(word >> 4*i) & 0x000f000f`` yields the adjacent pair ``(k+2i, k+2i+1)`` which is what
           one half of an ``mma.m16n8k16`` B fragment wants.  Rows past N are zero.
  params   ``[tiles][kblocks][128/group][128 channels][2]`` = (scale, zero point) in the dtype of
           the canonical scales (zero point 0 when the weight is symmetric).

``b200_w4_lanes_v1`` (cluster split-K decode GEMV, the default decode layout):
  weights  uint8 ``[N/128 tiles][K/128 kblocks][4 warps][2 row tiles][2 halves][32 lanes][16 bytes]``
           Lane ``4*r + c`` of (warp ``w``, row tile ``t``) holds, for the eight ``mma.m16n8k16`` steps
           ``j`` of the block, one 32-bit word each: words 0..3 in half 0, words 4..7 in half 1 (a
           warp-wide 16-byte load of one half is 512 contiguous bytes).  Its nibble positions 0..7 carry channels
           ``128*tile + 32*w + 16*t + r + (0,8,0,8,0,8,0,8)`` at ``k = 128*kblock + 32*(j//2) + 8*c +
           4*(j%2) + (0,0,2,2,1,1,3,3)``: ``(word >> 4*i) & 0x000f000f`` is register ``i`` of the A
           fragment, and the 16 bytes of activations a lane needs for two steps are contiguous.
           Codes are unsigned; two's-complement nibbles are stored as ``code + 8``.  Rows past N are zero.
  params   ``[2 or 1][tiles][kblocks][128/group][4 warps][8 r][4]``: plane 0 the scales, plane 1 the zero
           points (absent for symmetric weights) of the four channels ``32*w + 16*t + 8*h + r`` a lane's
           accumulators belong to, index ``2*t + h``; the two planes are passed to the kernel as
           separate arrays.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .errors import XQTBackendError

TILE_ROWS = 128
KBLOCK = 128
_NIBBLE_E = (0, 2, 4, 6, 1, 3, 5, 7)


@dataclass(frozen=True)
class TiledW4:
    """Decode execution layout of one W4 layer (see module docstring).

    ``layout`` is ``"tile128"`` (weights ``[tiles, kblocks, 16, 32, 16]``, lane-major, for the
    stream-K mma.sync decode kernel), ``"rows128"`` (weights ``[tiles, kblocks, 4, 128, 16]``, one
    16-byte chunk of 32 K per channel, for the tcgen05 decode kernel whose threads each own a
    channel) or ``"lanes"`` (weights ``[tiles, kblocks, 4, 2, 2, 32, 16]``, params
    ``[planes, tiles, kblocks, 128/group, 4, 8, 4]``, for the cluster split-K decode kernel).
    """

    weights: torch.Tensor      # uint8 [tiles, kblocks, 16, 32, 16]
    params: torch.Tensor       # [tiles, kblocks, 128/group, 128, 2]
    n: int
    k: int
    group_size: int
    nibble_signed: bool
    has_zero_point: bool
    layout: str = "tile128"
    integer_zero_points: bool = True

    @property
    def tiles(self) -> int:
        return int(self.weights.shape[0])

    @property
    def nbytes(self) -> int:
        return self.weights.numel() + self.params.numel() * self.params.element_size()


def tile_w4(qweight: torch.Tensor, scales: torch.Tensor, zero_points: torch.Tensor | None, *,
            group_size: int, nibble_signed: bool, k: int | None = None) -> TiledW4:
    """canonical ``[N, K/2]`` bytes + ``[N, G]`` params -> :class:`TiledW4` (pure index shuffling)."""

    if qweight.ndim != 2 or qweight.dtype != torch.uint8:
        raise XQTBackendError("tile_w4 expects canonical uint8 [N, K/2] storage")
    n, padded_k = int(qweight.shape[0]), int(qweight.shape[1]) * 2
    k = padded_k if k is None else int(k)
    if k != padded_k or k % KBLOCK != 0:
        raise XQTBackendError("the B200 decode layout needs K == padded_K and K a multiple of 128")
    if group_size not in (32, 64, 128):
        raise XQTBackendError("group_size must be 32, 64 or 128")
    groups = k // group_size
    if tuple(scales.shape) != (n, groups):
        raise XQTBackendError(f"scales must be [{n},{groups}]")
    tiles, kblocks, per_block = -(-n // TILE_ROWS), k // KBLOCK, KBLOCK // group_size
    rows = tiles * TILE_ROWS
    codes = torch.stack((qweight & 0x0F, qweight >> 4), dim=-1).reshape(n, k)
    if rows != n:
        codes = torch.nn.functional.pad(codes, (0, 0, 0, rows - n))
    # [tile, ntile, g, kblock, w, t, e]
    c = codes.reshape(tiles, 16, 8, kblocks, 4, 4, 8)
    c = c[..., list(_NIBBLE_E)]
    packed = c[..., 0::2] | (c[..., 1::2] << 4)                   # [tile, ntile, g, kblock, w, t, 4 bytes]
    weights = packed.permute(0, 3, 1, 2, 5, 4, 6).contiguous()    # [tile, kblock, ntile, g, t, w, byte]
    weights = weights.reshape(tiles, kblocks, 16, 32, 16)

    def tiled(param: torch.Tensor) -> torch.Tensor:
        p = param
        if rows != n:
            p = torch.nn.functional.pad(p, (0, 0, 0, rows - n))
        return p.reshape(tiles, TILE_ROWS, kblocks, per_block).permute(0, 2, 3, 1)   # [tile, kblock, sub, row]

    zeros = torch.zeros_like(scales) if zero_points is None else zero_points.to(scales.dtype)
    params = torch.stack((tiled(scales), tiled(zeros)), dim=-1).contiguous()
    return TiledW4(weights=weights, params=params, n=n, k=k, group_size=int(group_size),
                   nibble_signed=bool(nibble_signed), has_zero_point=zero_points is not None)


def rows_w4(qweight: torch.Tensor, scales: torch.Tensor, zero_points: torch.Tensor | None, *,
            group_size: int, nibble_signed: bool, k: int | None = None) -> TiledW4:
    """canonical tensors -> ``b200_w4_rows128_v1``: weights ``[tile][kblock][chunk][channel][16 B]``.

    Chunk ``c`` of channel ``r`` holds ``k = 128*kblock + 32*c .. +31``; inside each 32-bit word the
    nibble positions carry ``e = 0,2,4,6,1,3,5,7`` (as in ``tile_w4``), so the pair extracted by
    ``(word >> 4i) & 0x000f000f`` is one 32-bit tensor-memory column of the tcgen05 A operand.
    """

    base = tile_w4(qweight, scales, zero_points, group_size=group_size, nibble_signed=nibble_signed, k=k)
    tiles, kblocks = base.tiles, base.k // KBLOCK
    # tile128 lane order is [ntile j][g][t] with words w; word w of lane (g,t) covers k = 32w + 8t + e.
    w = base.weights.reshape(tiles, kblocks, 16, 8, 4, 4, 4)          # [tile, kb, j, g, t, w, byte]
    # rows layout wants, per channel (8j+g), chunk c = 32-K run, inside it word index = t' (8-K runs in order)
    w = w.permute(0, 1, 5, 2, 3, 4, 6)                                 # [tile, kb, w(=chunk), j, g, t(=word), byte]
    weights = w.reshape(tiles, kblocks, 4, TILE_ROWS, 16).contiguous()
    integer = True
    if zero_points is not None:
        z = zero_points.to(torch.float32)
        integer = bool((z == z.round()).all()) and bool((z >= 0).all()) and bool((z <= 119).all())
    return TiledW4(weights=weights, params=base.params, n=base.n, k=base.k, group_size=base.group_size,
                   nibble_signed=base.nibble_signed, has_zero_point=base.has_zero_point, layout="rows128",
                   integer_zero_points=integer)


_LANE_SLOT_ORDER = (0, 2, 1, 3)


def lanes_w4(qweight: torch.Tensor, scales: torch.Tensor, zero_points: torch.Tensor | None, *,
             group_size: int, nibble_signed: bool, k: int | None = None) -> TiledW4:
    """canonical tensors -> ``b200_w4_lanes_v1`` (see module docstring); pure index shuffling."""

    if qweight.ndim != 2 or qweight.dtype != torch.uint8:
        raise XQTBackendError("lanes_w4 expects canonical uint8 [N, K/2] storage")
    n, padded_k = int(qweight.shape[0]), int(qweight.shape[1]) * 2
    k = padded_k if k is None else int(k)
    if k != padded_k or k % KBLOCK != 0:
        raise XQTBackendError("the B200 decode layout needs K == padded_K and K a multiple of 128")
    if group_size not in (64, 128):
        raise XQTBackendError("the lanes layout serves group_size 64 or 128")
    groups = k // group_size
    if tuple(scales.shape) != (n, groups):
        raise XQTBackendError(f"scales must be [{n},{groups}]")
    tiles, kblocks, per_block = -(-n // TILE_ROWS), k // KBLOCK, KBLOCK // group_size
    rows = tiles * TILE_ROWS
    codes = torch.stack((qweight & 0x0F, qweight >> 4), dim=-1).reshape(n, k)
    if nibble_signed:
        codes = codes ^ 8
    if rows != n:
        codes = torch.nn.functional.pad(codes, (0, 0, 0, rows - n))
    # channel = 32w + 16t + 8h + r; k = 128kb + 32q + 8c + 4jj + slot
    c = codes.reshape(tiles, 4, 2, 2, 8, kblocks, 4, 4, 2, 4)      # [T, w, t, h, r, kb, q, c, jj, slot]
    c = c.permute(0, 5, 1, 2, 4, 7, 6, 8, 9, 3)                     # [T, kb, w, t, r, c, q, jj, slot, h]
    c = c[..., list(_LANE_SLOT_ORDER), :]
    nib = c.reshape(tiles, kblocks, 4, 2, 32, 8, 8)                 # [.., lane, word j, nibble p = 2*slot' + h]
    by = (nib[..., 0::2] | (nib[..., 1::2] << 4)).reshape(tiles, kblocks, 4, 2, 32, 2, 16)   # [.., lane, half, 16 B]
    weights = by.permute(0, 1, 2, 3, 5, 4, 6).contiguous()          # [tile, kb, warp, row tile, half, lane, 16 B]

    def laned(param: torch.Tensor) -> torch.Tensor:
        q = param
        if rows != n:
            q = torch.nn.functional.pad(q, (0, 0, 0, rows - n))
        q = q.reshape(tiles, 4, 2, 2, 8, kblocks, per_block)       # [T, w, t, h, r, kb, sub]
        return q.permute(0, 5, 6, 1, 4, 2, 3).reshape(tiles, kblocks, per_block, 4, 8, 4)

    planes = (laned(scales),) if zero_points is None else (laned(scales), laned(zero_points.to(scales.dtype)))
    params = torch.stack(planes, dim=0).contiguous()
    return TiledW4(weights=weights, params=params, n=n, k=k, group_size=int(group_size),
                   nibble_signed=bool(nibble_signed), has_zero_point=zero_points is not None, layout="lanes")


def _unlane_w4(tiled: TiledW4) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor | None]:
    tiles, kblocks, per_block = tiled.tiles, tiled.k // KBLOCK, KBLOCK // tiled.group_size
    w = tiled.weights.permute(0, 1, 2, 3, 5, 4, 6).reshape(tiles, kblocks, 4, 2, 32, 8, 4)
    nib = torch.stack((w & 0x0F, w >> 4), dim=-1).reshape(tiles, kblocks, 4, 2, 8, 4, 4, 2, 4, 2)
    #                                                      [T, kb, w, t, r, c, q, jj, slot', h]
    inverse = [list(_LANE_SLOT_ORDER).index(e) for e in range(4)]
    nib = nib[..., inverse, :]
    codes = nib.permute(0, 2, 3, 9, 4, 1, 6, 5, 7, 8).reshape(tiles * TILE_ROWS, tiled.k)[: tiled.n]
    if tiled.nibble_signed:
        codes = codes ^ 8
    qweight = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    def unlaned(plane: torch.Tensor) -> torch.Tensor:
        q = plane.reshape(tiles, kblocks, per_block, 4, 8, 2, 2)              # [T, kb, sub, w, r, t, h]
        return q.permute(0, 3, 5, 6, 4, 1, 2).reshape(tiles * TILE_ROWS, -1)[: tiled.n].contiguous()

    scales = unlaned(tiled.params[0])
    zeros = unlaned(tiled.params[1]) if tiled.has_zero_point else None
    return qweight, scales, zeros


def untile_w4(tiled: TiledW4) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor | None]:
    """Inverse of :func:`tile_w4` (used by the round-trip test and by checkpoint export)."""

    if tiled.layout == "lanes":
        return _unlane_w4(tiled)
    tiles, kblocks = tiled.tiles, tiled.k // KBLOCK
    weights = tiled.weights
    if tiled.layout == "rows128":
        weights = weights.reshape(tiles, kblocks, 4, 16, 8, 4, 4).permute(0, 1, 3, 4, 5, 2, 6)
    w = weights.reshape(tiles, kblocks, 16, 8, 4, 4, 4)           # [tile, kblock, ntile, g, t, w, byte]
    w = w.permute(0, 2, 3, 1, 5, 4, 6)                            # [tile, ntile, g, kblock, w, t, byte]
    nib = torch.stack((w & 0x0F, w >> 4), dim=-1).reshape(*w.shape[:-1], 8)   # nibble positions 0..7
    inverse = [list(_NIBBLE_E).index(e) for e in range(8)]
    codes = nib[..., inverse].reshape(tiles * TILE_ROWS, tiled.k)[: tiled.n]
    qweight = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    p = tiled.params.permute(0, 3, 1, 2, 4).reshape(tiles * TILE_ROWS, -1, 2)[: tiled.n]
    scales = p[..., 0].contiguous()
    zeros = p[..., 1].contiguous() if tiled.has_zero_point else None
    return qweight, scales, zeros


__all__ = ["KBLOCK", "TILE_ROWS", "TiledW4", "lanes_w4", "rows_w4", "tile_w4", "untile_w4"]
