"""Oracle for the ConvRot-style W8A8 int8 linear.  Test infrastructure only.

Weight side (offline): rotate the rows of ``W[N,K]`` block-wise, then symmetric
per-output-channel int8 with ``absmax`` clamped at ``eps``:
``scale = max(absmax/127, eps)``, ``q = clamp(round(w/scale), -127, 127)``
(xqt/compression/quant/quantizers/convrot_int8.py:361-400,1528-1541).

Activation side (every call): rotate, round to the activation dtype (every
reference variant quantises the rotated activation in its storage dtype:
convrot_int8.py:432-452, convrot_w8a8_sm89_kernel.cu:57-333), then dynamic
per-token int8 exactly as the GEMM-contract reference does:
``scale = max(amax, 1e-8)/127``, ``q = clamp(round(x/scale), -128, 127)``
(xqt/kernels/ops/gemm/quantize.py:60-107).

Product: the contract reference dequantises both sides and multiplies in fp32
(xqt/kernels/ops/gemm/reference.py:278-323,527); :func:`gemm_integer` is the
algebraically equal integer form ``int32(q_a @ q_w.T) * s_a[m] * s_w[n]`` a
tensor-core kernel evaluates.  They agree to fp32 summation order.
"""

from __future__ import annotations

import torch

from . import rotation
from .w4a16 import epilogue


def quantize_weight_per_channel(weight_rot: torch.Tensor, *, eps: float = 1e-6):
    """-> (q int8 [N,K], scale fp32 [N])  (convrot_int8.py:1528-1541, mse_clip off)."""

    w = weight_rot.to(torch.float32)
    absmax = w.abs().amax(dim=1, keepdim=True).clamp_min(float(eps))
    scale = (absmax / 127.0).clamp_min(float(eps))
    q = torch.round(w / scale).clamp(-127, 127).to(torch.int8)
    return q, scale.reshape(-1)


def quantize_act_per_token(x_rot: torch.Tensor):
    """-> (q int8 [M,K], scale fp32 [M,1])  (quantize.py:75-107, activation_dynamic/per_token)."""

    v = x_rot.to(torch.float32)
    scale = v.abs().amax(dim=1, keepdim=True).clamp_min(1e-8) / 127.0
    q = torch.round(v / scale.clamp_min(1e-8)).clamp(-128, 127).to(torch.int8)
    return q, scale


def quantize_act_per_tensor(x: torch.Tensor, *, eps: float = 1e-6):
    """-> (q int8 [M,K], scale fp32 scalar): ``Int8MmaLinear`` (xqt/contracts/int8_mma.py:135-149,317-319):
    ``scale = max(absmax, eps)/127``, ``q = clamp(round(x/scale), -127, 127)``."""

    v = x.to(torch.float32)
    scale = (v.reshape(-1).abs().amax().clamp_min(float(eps)) / 127.0).reshape(())
    q = torch.round(v / scale).clamp(-127, 127).to(torch.int8)
    return q, scale


def gemm_reference(q_a, s_a, q_w, s_w, *, bias=None, out_dtype=torch.bfloat16):
    """Dequantise both operands, fp32 matmul (reference.py:511-533)."""

    a = q_a.to(torch.float32) * s_a.to(torch.float32).reshape(-1, 1)
    w = q_w.to(torch.float32) * s_w.to(torch.float32).reshape(-1, 1)
    return epilogue(a @ w.transpose(0, 1), bias=bias, out_dtype=out_dtype)


def gemm_integer(q_a, s_a, q_w, s_w, *, bias=None, out_dtype=torch.bfloat16):
    """Exact integer accumulation, then ``acc * (s_a[m] * s_w[n])`` in fp32."""

    # int8 x int8 products summed over K fit in float64 exactly (|acc| < 2^53).
    acc = (q_a.to(torch.float64) @ q_w.to(torch.float64).transpose(0, 1)).to(torch.float32)
    scale = s_a.to(torch.float32).reshape(-1, 1) * s_w.to(torch.float32).reshape(1, -1)
    return epilogue(acc * scale, bias=bias, out_dtype=out_dtype)


def linear(
    x: torch.Tensor,
    q_w: torch.Tensor,
    s_w: torch.Tensor,
    *,
    rot_block: int = 256,
    rot_kind: str = "regular",
    signs: torch.Tensor | None = None,
    bias=None,
    integer: bool = False,
):
    """Full forward: rotate -> per-token int8 -> GEMM -> fp32 dequant epilogue."""

    x_rot = rotation.rotate_fht(x, kind=rot_kind, block=rot_block, signs=signs)
    q_a, s_a = quantize_act_per_token(x_rot)
    fn = gemm_integer if integer else gemm_reference
    return fn(q_a, s_a, q_w, s_w, bias=bias, out_dtype=x.dtype)
