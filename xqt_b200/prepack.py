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
    """Decode execution layout of one W4 layer (see module docstring)."""

    weights: torch.Tensor      # uint8 [tiles, kblocks, 16, 32, 16]
    params: torch.Tensor       # [tiles, kblocks, 128/group, 128, 2]
    n: int
    k: int
    group_size: int
    nibble_signed: bool
    has_zero_point: bool

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


def untile_w4(tiled: TiledW4) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor | None]:
    """Inverse of :func:`tile_w4` (used by the round-trip test and by checkpoint export)."""

    tiles, kblocks = tiled.tiles, tiled.k // KBLOCK
    w = tiled.weights.reshape(tiles, kblocks, 16, 8, 4, 4, 4)     # [tile, kblock, ntile, g, t, w, byte]
    w = w.permute(0, 2, 3, 1, 5, 4, 6)                            # [tile, ntile, g, kblock, w, t, byte]
    nib = torch.stack((w & 0x0F, w >> 4), dim=-1).reshape(*w.shape[:-1], 8)   # nibble positions 0..7
    inverse = [list(_NIBBLE_E).index(e) for e in range(8)]
    codes = nib[..., inverse].reshape(tiles * TILE_ROWS, tiled.k)[: tiled.n]
    qweight = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    p = tiled.params.permute(0, 3, 1, 2, 4).reshape(tiles * TILE_ROWS, -1, 2)[: tiled.n]
    scales = p[..., 0].contiguous()
    zeros = p[..., 1].contiguous() if tiled.has_zero_point else None
    return qweight, scales, zeros


__all__ = ["KBLOCK", "TILE_ROWS", "TiledW4", "tile_w4", "untile_w4"]
