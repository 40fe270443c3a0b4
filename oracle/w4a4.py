"""Oracle for the W4A4 SVDQuant / ConvRot linear.  Test infrastructure only.

Weight side (offline), as xqt's SVD quantiser builds its composite artifact:
``U,S,Vh = svd(W)``; ``L1 = diag(sqrt(S_r)) Vh_r`` (down, ``[r,K]``),
``L2 = U_r diag(sqrt(S_r))`` (up, ``[N,r]``), ``R = W - L2 L1``
(xqt/analysis/svd_analysis.py:46-120); the residual is quantised per
(row, K group) as ``scale = absmax/7`` (1 for a zero group),
``q = clamp(round(r / (scale + 1e-12)), -8, 7)`` and stored as signed nibbles,
low nibble first (xqt/compression/quant/quantizers/svd.py:92-128,
xqt/contracts/packing_int4.py:23-29).

Forward, reference CPU semantics (activations NOT quantised):
``y = x @ dequant(R).T + (x @ L1.T) @ L2.T + bias``
(xqt/contracts/composite.py:187-202).

Forward, W4A4 semantics.  The reference has them only as CUDA
(gemm_w4a4.cuh:534-624: one scale per (token, 64-K group), ``absmax/7``;
gemm_base.cuh:367-446: every 64-K slab's int32 partial sum is multiplied by
``a_scale * w_scale`` and accumulated; lora.cuh:110-243: the low-rank branch is
taken from the same, unquantised, rotated activation).  PARITY UNPINNED for the
activation codes: no CPU code or stored vector of the reference fixes them.  The
restatement applies the reference's CPU per-token formula
``scale = max(amax/7, 1e-6)``, ``q = clamp(round(x/scale), -8, 7)``
(convrot_4bit.py:669-679) at that group granularity, in fp32, on the rotated
activation rounded to its storage dtype, and accumulates in fp32 (the sm_89
kernel accumulates in half precision; fp32 is what the contract here requires).
"""

from __future__ import annotations

import torch

from . import rotation
from .w4a16 import pack_nibbles, unpack_nibbles


def svd_split(weight: torch.Tensor, rank: int):
    """-> (L1 [r,K], L2 [N,r], residual [N,K]) in fp32 (svd_analysis.py:53-76,92-120)."""

    w = weight.to(torch.float32)
    u, s, vh = torch.linalg.svd(w, full_matrices=False)
    r = min(int(rank), min(w.shape) - 1)
    root = torch.sqrt(torch.clamp(s[:r], min=0.0))
    down = torch.diag(root) @ vh[:r, :]
    up = u[:, :r] @ torch.diag(root)
    return down, up, w - up @ down


def quantize_residual(residual: torch.Tensor, *, group_size: int):
    """-> (packed uint8 [N,K/2], scale fp32 [N,G])  (svd.py:92-128)."""

    n, k = residual.shape
    assert k % group_size == 0
    grouped = residual.to(torch.float32).reshape(n, k // group_size, group_size)
    absmax = grouped.abs().amax(dim=2, keepdim=True)
    scale = torch.where(absmax > 0, absmax / 7.0, torch.ones_like(absmax))
    codes = torch.clamp(torch.round(grouped / (scale + 1e-12)), -8, 7).to(torch.int8)
    return pack_nibbles(codes.reshape(n, k), signed=True), scale.squeeze(-1)


def dequantize_residual(packed: torch.Tensor, scale: torch.Tensor, *, group_size: int) -> torch.Tensor:
    """(composite.py:160-172)"""

    n = packed.shape[0]
    codes = unpack_nibbles(packed, packed.shape[1] * 2, signed=True)
    return (codes.reshape(n, -1, group_size) * scale.to(torch.float32).unsqueeze(-1)).reshape(n, -1)


def composite_forward(x, packed, scale, down, up, *, group_size: int, bias=None):
    """``CompositeAddLinear.forward`` (composite.py:187-202): everything in ``x.dtype``."""

    dtype = x.dtype
    w = dequantize_residual(packed, scale, group_size=group_size).to(dtype)
    out = torch.nn.functional.linear(x, w)
    out = out + torch.nn.functional.linear(torch.nn.functional.linear(x, down.to(dtype)), up.to(dtype))
    if bias is not None:
        out = out + bias.to(dtype)
    return out


def quantize_act_groups(x_rot: torch.Tensor, *, group_size: int = 64):
    """-> (codes int8 [M,K], scale fp32 [M,G]); see the module docstring."""

    m, k = x_rot.shape
    assert k % group_size == 0
    grouped = x_rot.to(torch.float32).reshape(m, k // group_size, group_size)
    scale = torch.clamp(grouped.abs().amax(dim=2, keepdim=True) / 7.0, min=1e-6)
    codes = torch.clamp(torch.round(grouped / scale), -8, 7).to(torch.int8)
    return codes.reshape(m, k), scale.squeeze(-1)


def w4a4_forward(
    x: torch.Tensor,
    packed: torch.Tensor,
    w_scale: torch.Tensor,
    down: torch.Tensor,
    up: torch.Tensor,
    *,
    group_size: int = 64,
    rot_kind: str | None = "sylvester",
    rot_block: int = 128,
    signs: torch.Tensor | None = None,
    bias=None,
    return_parts: bool = False,
    act_group_size: int | None = None,
):
    """rotate -> group int4 activations -> int GEMM with per-slab scales -> + low rank -> + bias.

    ``act_group_size`` (default: ``group_size``) is the span of one activation scale; ``K`` gives the
    per-token form, whose one scale per row is applied to every weight slab.

    ``down`` / ``up`` are used at the precision they are given in (bf16 factors
    are upcast to fp32 exactly).  Output is cast once to ``x.dtype``.
    """

    if rot_kind is None:
        x_rot = x
    else:
        x_rot = rotation.rotate_fht(x, kind=rot_kind, block=rot_block, signs=signs)
    act_group = int(act_group_size or group_size)
    q_a, s_a = quantize_act_groups(x_rot, group_size=act_group)
    m, k = q_a.shape
    n = packed.shape[0]
    groups = k // group_size
    assert act_group % group_size == 0
    s_a = s_a.repeat_interleave(act_group // group_size, dim=1)
    q_w = unpack_nibbles(packed, k, signed=True)
    # Per-slab integer partial sums are exact in fp32 (|sum| <= 64*8*8 = 4096).
    qa = q_a.to(torch.float32).reshape(m, groups, group_size)
    qw = q_w.reshape(n, groups, group_size)
    acc = torch.zeros((m, n), dtype=torch.float32)
    sw = w_scale.to(torch.float32)
    for g in range(groups):
        partial = qa[:, g] @ qw[:, g].transpose(0, 1)
        acc += partial * (s_a[:, g].reshape(m, 1) * sw[:, g].reshape(1, n))
    low = x_rot.to(torch.float32) @ down.to(torch.float32).transpose(0, 1)
    out = acc + low @ up.to(torch.float32).transpose(0, 1)
    if bias is not None:
        out = out + bias.to(torch.float32)
    out = out.to(x.dtype)
    if return_parts:
        return out, {"x_rot": x_rot, "q_a": q_a, "s_a": s_a, "low": low}
    return out


def w4a4_forward_dequant(x, packed, w_scale, down, up, *, group_size=64, rot_kind="sylvester",
                         rot_block=128, signs=None, bias=None):
    """Same result as :func:`w4a4_forward` written as one dense fp32 product
    ``(q_a s_a) @ (q_w s_w).T`` (the form used for the full-size CPU baseline)."""

    x_rot = x if rot_kind is None else rotation.rotate_fht(x, kind=rot_kind, block=rot_block, signs=signs)
    q_a, s_a = quantize_act_groups(x_rot, group_size=group_size)
    a = q_a.to(torch.float32) * s_a.repeat_interleave(group_size, dim=1)
    w = dequantize_residual(packed, w_scale, group_size=group_size)
    out = a @ w.transpose(0, 1)
    out = out + (x_rot.to(torch.float32) @ down.to(torch.float32).t()) @ up.to(torch.float32).t()
    if bias is not None:
        out = out + bias.to(torch.float32)
    return out.to(x.dtype)
