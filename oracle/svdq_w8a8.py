"""Oracle for the SVDQuant W8A8 linear (int8 x int8 with a low-rank branch).  Test infrastructure only.

Parity unpinned: the reference implements this path only as CUDA kernels
(xqt/kernels/jit/csrc/quantization/svdq_w8a8_sm89_kernel.cu over jit/include/nunchaku/gemm_w8a8.cuh and lora.cuh,
driven by xqt/kernels/ops/_impl/cute/svdq_w8a8_sm89.py:158-312) and ships no golden vectors for it; this file restates
those kernels' arithmetic on the CPU and is checked against nothing but itself.

Weight side (svdq_w8a8_sm89.py:182-193): per output channel ``scale = bf16(absmax/127)``, 1 where the row is zero;
``q = clamp(rint(w / scale), -128, 127)`` (the kernel multiplies by an approximate reciprocal of the scale,
gemm_w8a8.cuh:74-125; here the IEEE quotient).

Activation side, every call (gemm_w8a8.cuh:236-262): per token ``scale = T(absmax/127)`` in the activation dtype T
(0 for an all-zero token, whose codes are 0), ``q = clamp(rint(x / scale), -128, 127)``.

Product (svdq_w8a8_sm89_kernel.cu:617-700): ``y = int32(q_a q_w^T) * s_a[m] * s_w[n] + bias[n] + lora_scale * la up^T``
with ``la = x down^T`` (fp32); ``lora_scale * la`` is rounded to T before the up projection (the kernel scales the fp32
activations and packs them to T for its MMA, lora.cuh:147-170), fp32 sums, one rounding of ``y`` to T.
"""

from __future__ import annotations

import torch


def quantize_weight(weight: torch.Tensor):
    """bf16/fp16 ``[N,K]`` -> (q int8 ``[N,K]``, scale fp32 ``[N]`` holding T-representable values)."""

    w = weight.to(torch.float32)
    amax = w.abs().amax(dim=1)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax)).to(weight.dtype).to(torch.float32)
    q = torch.round(w / scale[:, None]).clamp(-128, 127).to(torch.int8)
    return q, scale


def quantize_act(x: torch.Tensor):
    """T ``[M,K]`` -> (q int8 ``[M,K]``, scale fp32 ``[M]``)."""

    xf = x.to(torch.float32)
    amax = xf.abs().amax(dim=1)
    scale = (amax / 127.0).to(x.dtype).to(torch.float32)
    safe = torch.where(scale > 0, scale, torch.ones_like(scale))
    q = torch.round(xf / safe[:, None]).clamp(-128, 127).to(torch.int8)
    return q, scale


def forward(x: torch.Tensor, q_w: torch.Tensor, s_w: torch.Tensor, down: torch.Tensor | None, up: torch.Tensor | None,
            bias: torch.Tensor | None = None, lora_scale: float = 1.0, return_parts: bool = False):
    q_a, s_a = quantize_act(x)
    acc = (q_a.to(torch.float64) @ q_w.to(torch.float64).t()).to(torch.float32)        # exact: |acc| < 2^31
    y = acc * (s_a[:, None] * s_w[None, :])
    if bias is not None:
        y = y + bias.to(torch.float32)[None, :]
    if down is not None:
        la = x.to(torch.float32) @ down.to(torch.float32).t()
        low = (la * float(lora_scale)).to(x.dtype).to(torch.float32) @ up.to(torch.float32).t()
        y = y + low
    out = y.to(x.dtype)
    return (out, {"q_a": q_a, "s_a": s_a}) if return_parts else out
