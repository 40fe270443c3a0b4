"""ConvRot-style W8A8 int8 linear on B200.

Python surface of xqt's native op (xqt/kernels/ops/_impl/cute/convrot_w8a8_sm89.py:154-500):
``pack_convrot_w8a8_linear`` -> ``PackedConvRotW8A8Linear``; ``convrot_w8a8_linear(inputs, packed,
rotated_input_features=..., rot_size=...)``; ``bind_convrot_w8a8_linear``.  The packed tensor
contents are backend-private; here the weight is simply int8 ``[N, K]`` K-major (what the TMA
descriptor of the tcgen05 GEMM reads), produced from the artifact's transposed ``qweight_t [K, N]``
(xqt/compression/quant/quantizers/convrot_int8.py:361-400).

Per call: one prologue kernel (rotate, round to the activation dtype, per-token int8) and one
tcgen05 ``kind::i8`` GEMM whose epilogue applies ``a_scale[m] * w_scale[n]`` (+ bias) in fp32.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import native
from ..errors import XQTBackendError
from ..quantize import Rotation, regular_rotation
from .activation import rotate_quantize


@dataclass(frozen=True)
class PackedConvRotW8A8Linear:
    qweight: torch.Tensor          # int8 [N, padded_K], K-major
    weight_scales: torch.Tensor    # fp32 [N]
    bias: torch.Tensor | None      # fp32 [N]
    input_features: int
    output_features: int
    padded_input_features: int
    dtype: torch.dtype


def pack_convrot_w8a8_linear(qweight_t: torch.Tensor, weight_scale: torch.Tensor, bias: torch.Tensor | None = None,
                             *, dtype: torch.dtype = torch.bfloat16,
                             input_features: int | None = None) -> PackedConvRotW8A8Linear:
    """``qweight_t`` is the artifact's int8 ``[padded_K, N]`` buffer, ``weight_scale`` its fp32 ``[N]``."""

    if qweight_t.ndim != 2 or qweight_t.dtype != torch.int8:
        raise XQTBackendError("ConvRot W8A8 qweight_t must be int8 [K, N]")
    if dtype not in (torch.float16, torch.bfloat16):
        raise XQTBackendError("ConvRot W8A8 supports fp16 or bf16 activations")
    kp, n = int(qweight_t.shape[0]), int(qweight_t.shape[1])
    if weight_scale.numel() != n:
        raise XQTBackendError("ConvRot W8A8 weight_scale must have N elements")
    if kp % 16 or n % 8:
        raise XQTBackendError("ConvRot W8A8 on B200 needs padded K % 16 == 0 and N % 8 == 0")
    device = qweight_t.device
    return PackedConvRotW8A8Linear(
        qweight=qweight_t.t().contiguous(), weight_scales=weight_scale.reshape(-1).to(torch.float32).contiguous(),
        bias=None if bias is None else bias.reshape(-1).to(device=device, dtype=torch.float32).contiguous(),
        input_features=kp if input_features is None else int(input_features), output_features=n,
        padded_input_features=kp, dtype=dtype)


def w8a8_gemm(codes: torch.Tensor, act_scale: torch.Tensor, packed: PackedConvRotW8A8Linear,
              out: torch.Tensor | None = None) -> torch.Tensor:
    m, k = int(codes.shape[0]), int(codes.shape[1])
    n = packed.output_features
    device = codes.device
    if codes.dtype != torch.int8 or k != packed.padded_input_features or not codes.is_contiguous():
        raise XQTBackendError("W8A8 GEMM: activation codes must be contiguous int8 [M, padded_K]")
    if packed.qweight.device != device:
        raise XQTBackendError("W8A8 GEMM: weight and activation must share a device")
    if out is None:
        out = torch.empty((m, n), device=device, dtype=packed.dtype)
    if m == 0:
        return out
    scratch = native.workspace(device, 256, "gemm")
    with torch.cuda.device(device):
        code = native.library().xqt_b200_w8a8_gemm(
            codes.data_ptr(), packed.qweight.data_ptr(), act_scale.data_ptr(), packed.weight_scales.data_ptr(),
            native.ptr(packed.bias), out.data_ptr(), m, n, k, native.DTYPE_CODE[packed.dtype], scratch.data_ptr(),
            scratch.numel(), native.stream_handle(device))
    native.check(code, "xqt_b200_w8a8_gemm")
    return out


def convrot_w8a8_linear(inputs: torch.Tensor, packed: PackedConvRotW8A8Linear, *,
                        rotated_input_features: bool = False, rot_size: int = 256,
                        rotation: Rotation | None = None, workspace=None) -> torch.Tensor:
    """Full forward.  ``rotated_input_features=True`` means the caller already rotated the input
    (the rotation is skipped, the rounding and quantisation are not)."""

    del workspace  # scratch is managed per stream by xqt_b200.native
    if inputs.shape[-1] != packed.input_features:
        raise XQTBackendError("ConvRot W8A8 input trailing dimension does not match input_features")
    if inputs.dtype != packed.dtype:
        raise XQTBackendError("ConvRot W8A8 input dtype disagrees with the packed layer")
    x = inputs.reshape(-1, packed.input_features)
    if packed.padded_input_features != packed.input_features:
        x = torch.nn.functional.pad(x, (0, packed.padded_input_features - packed.input_features))
    if rotated_input_features:
        rot = None
    else:
        rot = rotation if rotation is not None else regular_rotation(int(rot_size))
    codes, scales = rotate_quantize(x, rot, bits=8)
    out = w8a8_gemm(codes, scales, packed)
    return out.reshape(*inputs.shape[:-1], packed.output_features)


def bind_convrot_w8a8_linear(packed: PackedConvRotW8A8Linear, *, rows: int, rot_size: int = 256,
                             rotated_input_features: bool = False, rotation: Rotation | None = None):
    """Closure for a fixed row count (cf. convrot_w8a8_sm89.py:441-500)."""

    def run(inputs: torch.Tensor) -> torch.Tensor:
        if inputs.reshape(-1, packed.input_features).shape[0] != rows:
            raise XQTBackendError("bound ConvRot W8A8 call: row count mismatch")
        return convrot_w8a8_linear(inputs, packed, rotated_input_features=rotated_input_features, rot_size=rot_size,
                                   rotation=rotation)

    return run


__all__ = ["PackedConvRotW8A8Linear", "bind_convrot_w8a8_linear", "convrot_w8a8_linear", "pack_convrot_w8a8_linear",
           "w8a8_gemm"]
