"""Operator-stage W4 pattern ``gemm_int4_dequant`` on B200.

xqt's operator stage describes a weight-only int4 linear by the pattern contract
``gemm_int4_dequant(a, b_packed, b_scale, b_zero, bias, *, group_size, activation)``
(xqt/kernels/ops/_impl/triton/gemm.py:262-314): ``b_packed`` uint8 ``[N, K/2]`` holds two's-complement
nibbles (low nibble = even k), ``b_scale`` is ``[N, G]`` or ``[N, G, 1]``, and -- unlike the GEMM
contract -- the zero is in REAL units and applied after the scale: ``w = scale * code - zero``.

That is ``scale * (code - zero / scale)``: the same kernels serve it with the (generally fractional)
zero point ``zero / scale``, which is why the decode kernel and the two-pass GEMM take any real zero
point.  The epilogue activation of the contract (relu / gelu / silu) goes to the kernels' own epilogue.
"""

from __future__ import annotations

import torch

from ..errors import XQTBackendError
from ..weakid import WeakIdDict
from .w4a16 import bind_w4a16_decode, prepare_decode, w4a16_linear

_layouts = WeakIdDict()      # b_packed tensor -> (versions, zero points, decode layout, bound callables)


def _zero_points(b_scale: torch.Tensor, b_zero: torch.Tensor | None) -> torch.Tensor | None:
    if b_zero is None:
        return None
    zero = b_zero.squeeze(-1) if b_zero.ndim == 3 and b_zero.shape[2] == 1 else b_zero
    if zero.shape != b_scale.shape:
        raise XQTBackendError("gemm_int4_dequant: b_zero must have the shape of b_scale")
    return zero.to(torch.float32) / b_scale


def gemm_int4_dequant(a: torch.Tensor, b_packed: torch.Tensor, b_scale: torch.Tensor, b_zero: torch.Tensor | None = None,
                      bias: torch.Tensor | None = None, *, group_size: int = 128, activation: str | None = None) -> torch.Tensor:
    """``act(a @ (scale * code - zero)^T + bias)`` with fp32 accumulation, output in ``a.dtype``."""

    if a.ndim != 2 or a.dtype not in (torch.float16, torch.bfloat16) or not a.is_cuda:
        raise XQTBackendError("gemm_int4_dequant on B200 expects a CUDA rank-2 fp16/bf16 activation")
    if b_packed.ndim != 2 or b_packed.dtype != torch.uint8 or not b_packed.is_contiguous():
        raise XQTBackendError("gemm_int4_dequant: b_packed must be contiguous uint8 [N, K/2]")
    n, k = int(b_packed.shape[0]), int(b_packed.shape[1]) * 2
    if int(a.shape[1]) != k:
        raise XQTBackendError("gemm_int4_dequant: activation K does not match the packed weight")
    if group_size not in (32, 64, 128) or k % int(group_size):
        raise XQTBackendError("gemm_int4_dequant on B200 serves group sizes 32, 64, 128 that divide K")
    scale = b_scale.squeeze(-1) if b_scale.ndim == 3 and b_scale.shape[2] == 1 else b_scale
    if tuple(scale.shape) != (n, k // int(group_size)):
        raise XQTBackendError("gemm_int4_dequant: b_scale must be [N, K/group_size] (or with a trailing 1)")
    act = "none" if activation in (None, "none") else str(activation)
    if act not in ("none", "relu", "gelu", "silu"):
        raise XQTBackendError(f"gemm_int4_dequant: unsupported activation {activation!r}")
    versions = (b_packed._version, id(b_scale), b_scale._version, None if b_zero is None else (id(b_zero), b_zero._version))
    hit = _layouts.get(b_packed)
    if hit is None or hit["versions"] != versions:
        scale32 = scale.to(torch.float32).contiguous()
        zeros = _zero_points(scale32, b_zero)
        hit = {"versions": versions, "scale": scale32, "zeros": None if zeros is None else zeros.contiguous(),
               "tiled": None, "bound": {}, "keep": (b_scale, b_zero)}
        _layouts[b_packed] = hit
    m = int(a.shape[0])
    if m <= 16 and act == "none" and int(group_size) in (64, 128) and k % 128 == 0:
        if hit["tiled"] is None:
            hit["tiled"] = prepare_decode(b_packed, hit["scale"], hit["zeros"], group_size=int(group_size), nibble_signed=True,
                                          layout="lanes")
        run = hit["bound"].get((m, a.dtype, None if bias is None else id(bias)))
        if run is None:
            run = bind_w4a16_decode(hit["tiled"], rows=m, dtype=a.dtype, bias=bias)
            hit["bound"][(m, a.dtype, None if bias is None else id(bias))] = run
            hit.setdefault("bias_keep", []).append(bias)
        return run(a.contiguous())
    return w4a16_linear(a.contiguous(), b_packed, hit["scale"], hit["zeros"], bias, group_size=int(group_size),
                        nibble_signed=True, activation=act)


__all__ = ["gemm_int4_dequant"]
