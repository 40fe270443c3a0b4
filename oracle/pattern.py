"""Oracle for the operator-stage pattern ``gemm_int4_dequant``.  Test infrastructure only.

Restates ``gemm_int4_dequant_reference`` (xqt/kernels/ops/_impl/triton/gemm.py:262-314) and the
``gemm_reference`` epilogue it ends in: two's-complement nibbles (low nibble = even k),
``w = code * scale - zero`` per group (zero in real units), ``y = act(a @ w^T + bias)``.  The reference
evaluates in the activation dtype; here everything is fp32 and rounded once, the form the kernels are
compared with (the reference's own bf16 arithmetic is coarser than the 1e-3 bar).
"""

from __future__ import annotations

import torch

from .w4a16 import epilogue


def dequantize(b_packed: torch.Tensor, b_scale: torch.Tensor, b_zero: torch.Tensor | None, *, group_size: int) -> torch.Tensor:
    n, half = b_packed.shape
    k = half * 2
    low = (b_packed & 0x0F).to(torch.int16)
    high = ((b_packed >> 4) & 0x0F).to(torch.int16)
    codes = torch.stack((low, high), dim=-1).reshape(n, k)
    codes = torch.where(codes > 7, codes - 16, codes).to(torch.float32)
    scale = b_scale.squeeze(-1) if b_scale.ndim == 3 else b_scale
    w = codes.reshape(n, k // group_size, group_size) * scale.to(torch.float32).unsqueeze(-1)
    if b_zero is not None:
        zero = b_zero.squeeze(-1) if b_zero.ndim == 3 else b_zero
        w = w - zero.to(torch.float32).unsqueeze(-1)
    return w.reshape(n, k)


def gemm_int4_dequant(a, b_packed, b_scale, b_zero=None, bias=None, *, group_size=128, activation=None):
    w = dequantize(b_packed, b_scale, b_zero, group_size=group_size)
    return epilogue(a.to(torch.float32) @ w.t(), bias=bias, residual=None, activation=activation or "none", out_dtype=a.dtype)
