"""Oracle for the W4A16 group-wise int4 linear.  Test infrastructure only.

Follows xqt/kernels/ops/gemm/reference.py: the weight is decoded to fp32 as
``(code - zero_point) * scale`` with scales / zero points expanded along K by
``repeat_interleave(group_size)`` (reference.py:52-80,165-275), the product is
``fp32(A) @ fp32(W).T`` (reference.py:527), then bias and residual are added in
fp32, the activation applied and the result cast once (reference.py:362-390).
"""

from __future__ import annotations

import torch


def unpack_nibbles(qweight: torch.Tensor, k: int, *, signed: bool) -> torch.Tensor:
    """Low-nibble-first decode to fp32 values (layout.py:571-585)."""

    assert qweight.dtype == torch.uint8 and qweight.ndim == 2
    low = (qweight & 0x0F).to(torch.int16)
    high = (qweight >> 4).to(torch.int16)
    codes = torch.stack((low, high), dim=-1).reshape(qweight.shape[0], -1)[:, :k]
    if signed:
        codes = torch.where(codes >= 8, codes - 16, codes)
    return codes.to(torch.float32)


def pack_nibbles(codes: torch.Tensor, *, signed: bool) -> torch.Tensor:
    """Inverse of :func:`unpack_nibbles` (layout.py:80-109)."""

    wide = codes.to(torch.int16)
    if signed:
        wide = torch.where(wide < 0, wide + 16, wide)
    if wide.shape[1] % 2:
        wide = torch.nn.functional.pad(wide, (0, 1))
    wide = wide.to(torch.uint8)
    return (wide[:, 0::2] | (wide[:, 1::2] << 4)).contiguous()


def dequantize(
    qweight: torch.Tensor,
    scales: torch.Tensor,
    zero_points: torch.Tensor | None,
    *,
    k: int,
    padded_k: int,
    group_size: int,
    signed: bool,
) -> torch.Tensor:
    """``[N,K]`` fp32 weight: ``(code - zero) * scale`` (reference.py:263-271)."""

    values = unpack_nibbles(qweight, padded_k, signed=signed)
    scale = scales.to(torch.float32).repeat_interleave(group_size, dim=1)[:, :padded_k]
    if zero_points is not None:
        zero = zero_points.to(torch.float32).repeat_interleave(group_size, dim=1)[:, :padded_k]
        values = values - zero
    return (values * scale)[:, :k]


def epilogue(acc, *, bias=None, residual=None, activation="none", out_dtype=torch.bfloat16):
    """bias -> residual -> activation -> one cast (reference.py:362-390)."""

    out = acc
    if bias is not None:
        out = out + bias.to(torch.float32)
    if residual is not None:
        out = out + residual.to(torch.float32)
    if activation == "relu":
        out = torch.relu(out)
    elif activation == "gelu":
        out = torch.nn.functional.gelu(out)
    elif activation == "silu":
        out = torch.nn.functional.silu(out)
    return out.to(out_dtype)


def gemm(
    x: torch.Tensor,
    qweight: torch.Tensor,
    scales: torch.Tensor,
    zero_points: torch.Tensor | None,
    *,
    group_size: int,
    signed: bool,
    k: int | None = None,
    bias=None,
    residual=None,
    activation: str = "none",
    out_dtype: torch.dtype | None = None,
) -> torch.Tensor:
    """``reference_w4a16_gemm`` restated (reference.py:469-577)."""

    k = int(x.shape[1]) if k is None else k
    padded_k = int(qweight.shape[1]) * 2
    weight = dequantize(
        qweight, scales, zero_points, k=k, padded_k=padded_k, group_size=group_size, signed=signed
    )
    acc = x.to(torch.float32) @ weight.transpose(0, 1)
    return epilogue(
        acc, bias=bias, residual=residual, activation=activation, out_dtype=out_dtype or x.dtype
    )


def rtn_uint4(weight: torch.Tensor, *, group_size: int, param_dtype=torch.bfloat16):
    """Asymmetric round-to-nearest uint4, the input definition of the benchmark configs.

    xqt ships no asymmetric RTN quantiser (its own are symmetric signed,
    contracts/weight_only.py:40-274); unsigned codes with zero points reach its
    kernels through checkpoint import.  The definition used for the synthetic
    configs is, per (row, K group): ``s = (max - min) / 15`` rounded to
    ``param_dtype``, ``z = clamp(round(-min / s), 0, 15)``,
    ``q = clamp(round(w / s + z), 0, 15)``; a flat group gets ``s = 1``.
    Returns (qweight uint8 [N, K/2], scales [N, G], zero_points [N, G]).
    """

    n, k = weight.shape
    assert k % group_size == 0
    grouped = weight.to(torch.float32).reshape(n, k // group_size, group_size)
    low = grouped.amin(dim=2, keepdim=True)
    high = grouped.amax(dim=2, keepdim=True)
    scale = (high - low) / 15.0
    scale = torch.where(scale > 0, scale, torch.ones_like(scale))
    scale = scale.to(param_dtype).to(torch.float32)
    zero = torch.clamp(torch.round(-low / scale), 0, 15)
    codes = torch.clamp(torch.round(grouped / scale + zero), 0, 15).to(torch.uint8)
    return (
        pack_nibbles(codes.reshape(n, k), signed=False),
        scale.squeeze(-1).to(param_dtype),
        zero.squeeze(-1).to(param_dtype),
    )


def rtn_int4_symmetric(weight: torch.Tensor, *, group_size: int):
    """xqt's own weight-only RTN: ``scale = absmax / 7`` (1 for a zero group),
    ``q = clamp(round(w / scale), -8, 7)`` (contracts/packing_int4.py:62-91).
    Returns (qweight uint8 signed nibbles, scales fp32 [N, G])."""

    n, k = weight.shape
    assert k % group_size == 0
    grouped = weight.to(torch.float32).reshape(n, k // group_size, group_size)
    absmax = grouped.abs().amax(dim=2, keepdim=True)
    scale = torch.where(absmax > 0, absmax / 7.0, torch.ones_like(absmax))
    codes = torch.clamp(torch.round(grouped / scale), -8, 7).to(torch.int8)
    return pack_nibbles(codes.reshape(n, k), signed=True), scale.squeeze(-1)


def rel_l2(actual: torch.Tensor, expected: torch.Tensor) -> float:
    a = actual.detach().to("cpu", torch.float64)
    e = expected.detach().to("cpu", torch.float64)
    return float((a - e).norm() / e.norm().clamp_min(1e-30))
