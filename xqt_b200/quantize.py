"""Offline weight quantisers and rotation matrices that define the inputs of the path.

These are the producer side of the canonical artifacts (they run once per layer, in plain torch,
on whatever device the weight lives on); nothing here is on the per-token hot path.  Each follows
the xqt quantiser that writes the corresponding artifact:

* symmetric signed int4 RTN per K group ......... xqt/contracts/packing_int4.py:62-91
* SVD split + int4 residual ....................... xqt/analysis/svd_analysis.py:46-120,
                                                    xqt/compression/quant/quantizers/svd.py:92-128
* per-output-channel int8 after rotation .......... xqt/compression/quant/quantizers/convrot_int8.py:361-400,1528-1541
* regular (4^k) Hadamard blocks .................... xqt/compression/quant/quantizers/convrot_4bit.py:85-123
* randomized Sylvester Hadamard blocks ............. xqt/model/minicpm5_quarot.py:54-93
* asymmetric uint4 RTN with zero points: xqt has no such quantiser (unsigned codes reach it through
  AWQ checkpoint import); the definition below is the one the benchmark configurations state.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .contracts import PackedWeight, QuantSpec
from .layout import W4_LAYOUT, W8_LAYOUT, build_packed_weight, pack_int4_signed, pack_int4_unsigned


def _grouped(weight: torch.Tensor, group_size: int) -> tuple[torch.Tensor, int]:
    n, k = weight.shape
    padded_k = -(-k // group_size) * group_size
    w = weight.detach().to(torch.float32)
    if padded_k != k:
        w = torch.nn.functional.pad(w, (0, padded_k - k))
    return w.reshape(n, padded_k // group_size, group_size), padded_k


def w4_spec(*, group_size: int, symmetric: bool, dtype: str = "bf16") -> QuantSpec:
    return QuantSpec(
        weight_dtype="int4", activation_dtype=dtype, output_dtype=dtype, weight_granularity="groupwise",
        group_size=int(group_size), symmetric=symmetric, weight_zero_point=not symmetric,
        weight_scale_source="weight_offline", storage_layout=W4_LAYOUT, pack_version="xqt-w4a16-b200-v1",
    )


def quantize_w4_asymmetric(weight: torch.Tensor, *, group_size: int = 128,
                           param_dtype: torch.dtype = torch.bfloat16, dtype: str = "bf16") -> PackedWeight:
    """uint4 codes + zero points: ``s=(max-min)/15`` (rounded to ``param_dtype``),
    ``z=clamp(round(-min/s),0,15)``, ``q=clamp(round(w/s+z),0,15)``."""

    n, k = weight.shape
    grouped, padded_k = _grouped(weight, group_size)
    low, high = grouped.amin(dim=2, keepdim=True), grouped.amax(dim=2, keepdim=True)
    scale = (high - low) / 15.0
    scale = torch.where(scale > 0, scale, torch.ones_like(scale)).to(param_dtype).to(torch.float32)
    zero = torch.clamp(torch.round(-low / scale), 0, 15)
    codes = torch.clamp(torch.round(grouped / scale + zero), 0, 15).to(torch.uint8).reshape(n, padded_k)
    return build_packed_weight(
        pack_int4_unsigned(codes), logical_shape=(n, k), spec=w4_spec(group_size=group_size, symmetric=False, dtype=dtype),
        scales=scale.squeeze(-1).to(param_dtype).contiguous(), zero_points=zero.squeeze(-1).to(param_dtype).contiguous(),
        padded_k=padded_k,
    )


def quantize_w4_symmetric(weight: torch.Tensor, *, group_size: int = 128, dtype: str = "bf16") -> PackedWeight:
    """Signed int4, ``scale = absmax/7`` (1 for an all-zero group), fp32 scales."""

    n, k = weight.shape
    grouped, padded_k = _grouped(weight, group_size)
    absmax = grouped.abs().amax(dim=2, keepdim=True)
    scale = torch.where(absmax > 0, absmax / 7.0, torch.ones_like(absmax))
    codes = torch.clamp(torch.round(grouped / scale), -8, 7).to(torch.int8).reshape(n, padded_k)
    return build_packed_weight(
        pack_int4_signed(codes), logical_shape=(n, k), spec=w4_spec(group_size=group_size, symmetric=True, dtype=dtype),
        scales=scale.squeeze(-1).contiguous(), zero_points=None, padded_k=padded_k,
    )


# ----------------------------------------------------------------------------- rotations


def _is_power_of(value: int, base: int) -> bool:
    value = int(value)
    if value < 1:
        return False
    while value % base == 0:
        value //= base
    return value == 1


@dataclass(frozen=True)
class Rotation:
    """Block-diagonal Hadamard rotation ``x_block @ (H / sqrt(n) * signs)``.

    ``kind`` is ``"regular"`` (order 4^k, symmetric and self-inverse) or ``"sylvester"`` (order
    2^k).  ``column_scale`` is the fp32 vector ``signs / sqrt(block)`` the kernels multiply by
    after the add/sub butterflies.
    """

    kind: str
    block: int
    signs: torch.Tensor | None = None

    def __post_init__(self) -> None:
        if self.kind == "regular":
            if not _is_power_of(self.block, 4):
                raise ValueError("rot_size must be one or a power of four")
        elif self.kind == "sylvester":
            if not _is_power_of(self.block, 2):
                raise ValueError("Sylvester Hadamard order must be a power of two")
        else:
            raise ValueError(f"unknown rotation kind {self.kind!r}")
        if self.signs is not None and self.signs.numel() != self.block:
            raise ValueError("signs must have one entry per rotated column of a block")

    @property
    def column_scale(self) -> torch.Tensor:
        norm = torch.full((self.block,), 1.0 / math.sqrt(float(self.block)), dtype=torch.float64)
        if self.signs is not None:
            norm = norm * self.signs.detach().to("cpu", torch.float64)
        return norm.to(torch.float32)

    def matrix(self) -> torch.Tensor:
        if self.kind == "regular":
            base = torch.tensor(
                [[1.0, 1.0, 1.0, -1.0], [1.0, 1.0, -1.0, 1.0], [1.0, -1.0, 1.0, 1.0], [-1.0, 1.0, 1.0, 1.0]]
            )
            h = torch.ones((1, 1))
            while h.shape[0] < self.block:
                h = torch.kron(h, base)
        else:
            h = torch.ones((1, 1))
            while h.shape[0] < self.block:
                h = torch.cat((torch.cat((h, h), 1), torch.cat((h, -h), 1)), 0)
        h = (h.to(torch.float64) / math.sqrt(float(self.block))).to(torch.float32)
        if self.signs is not None:
            h = h * self.signs.detach().to("cpu", torch.float32).reshape(1, self.block)
        return h

    def apply(self, tensor: torch.Tensor) -> torch.Tensor:
        """Offline rotation of weight rows (fp32 matmul per block)."""

        k = tensor.shape[-1]
        if k % self.block:
            raise ValueError("rotated dimension must be a multiple of the rotation block")
        blocks = tensor.to(torch.float32).reshape(-1, k // self.block, self.block)
        return torch.matmul(blocks, self.matrix().to(tensor.device)).reshape(tensor.shape)


def regular_rotation(block: int = 256) -> Rotation:
    return Rotation("regular", int(block))


def randomized_rotation(block: int, seed: int) -> Rotation:
    """``H @ diag(signs)`` with the seeded +-1 draw of ``build_quarot_rotation``."""

    generator = torch.Generator(device="cpu").manual_seed(int(seed))
    bits = torch.randint(0, 2, (int(block),), generator=generator, dtype=torch.float64)
    kind = "regular" if _is_power_of(block, 4) else "sylvester"
    return Rotation(kind, int(block), bits.mul(2.0).sub(1.0).to(torch.float32))


# ----------------------------------------------------------------------------- W8A8 / W4A4 weights


def quantize_w8_per_channel(weight_rot: torch.Tensor, *, eps: float = 1e-6) -> tuple[torch.Tensor, torch.Tensor]:
    """-> (int8 ``[N,K]``, fp32 scale ``[N]``): ``scale=max(absmax/127, eps)``, codes in [-127,127]."""

    w = weight_rot.detach().to(torch.float32)
    absmax = w.abs().amax(dim=1, keepdim=True).clamp_min(float(eps))
    scale = (absmax / 127.0).clamp_min(float(eps))
    return torch.round(w / scale).clamp(-127, 127).to(torch.int8), scale.reshape(-1)


def w8_packed_weight(q: torch.Tensor, scale: torch.Tensor, dtype: str = "bf16") -> PackedWeight:
    spec = QuantSpec(
        weight_dtype="int8", activation_dtype="int8", output_dtype=dtype, weight_granularity="per_channel",
        activation_granularity="per_token", weight_scale_source="weight_offline",
        activation_scale_source="activation_dynamic", storage_layout=W8_LAYOUT, pack_version="xqt-w8a8-int8-v1",
    )
    n, k = q.shape
    return build_packed_weight(q, logical_shape=(n, k), spec=spec, scales=scale.reshape(n, 1).to(torch.float32))


def svd_split(weight: torch.Tensor, rank: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """-> (down ``[r,K]``, up ``[N,r]``, residual ``[N,K]``), all fp32."""

    w = weight.detach().to(torch.float32)
    u, s, vh = torch.linalg.svd(w, full_matrices=False)
    r = min(int(rank), min(w.shape) - 1)
    if r <= 0:
        raise ValueError(f"Rank {rank} is invalid for weight shape {tuple(w.shape)}")
    root = torch.sqrt(torch.clamp(s[:r], min=0.0))
    down, up = torch.diag(root) @ vh[:r, :], u[:, :r] @ torch.diag(root)
    return down, up, w - up @ down


def quantize_residual_int4(residual: torch.Tensor, *, group_size: int = 64) -> tuple[torch.Tensor, torch.Tensor, int]:
    """-> (packed uint8 ``[N,Kp/2]``, fp32 scale ``[N,G]``, padded K): ``scale=absmax/7`` (1 if zero),
    ``q=clamp(round(r/(scale+1e-12)),-8,7)``."""

    n, k = residual.shape
    group = max(1, min(int(group_size), int(k)))
    grouped, padded_k = _grouped(residual, group)
    absmax = grouped.abs().amax(dim=2, keepdim=True)
    scale = torch.where(absmax > 0, absmax / 7.0, torch.ones_like(absmax))
    codes = torch.clamp(torch.round(grouped / (scale + 1e-12)), -8, 7).to(torch.int8).reshape(n, padded_k)
    return pack_int4_signed(codes), scale.squeeze(-1).contiguous(), padded_k


__all__ = [
    "Rotation", "quantize_residual_int4", "quantize_w4_asymmetric", "quantize_w4_symmetric",
    "quantize_w8_per_channel", "randomized_rotation", "regular_rotation", "svd_split", "w4_spec",
    "w8_packed_weight",
]
