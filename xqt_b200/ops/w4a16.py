"""W4A16 linear on canonical ``xqt_int4_nk_v1`` tensors: the torch-facing call into the C ABI.

``w4a16_linear`` is registered as ``torch.ops.xqt_operator_opt.b200_w4a16_linear`` (xqt reserves
that namespace for its custom CUDA operators, xqt/kernels/wrappers/cuda_extension.py:20-85) with a
fake implementation for tracing; the real one only checks arguments, allocates the output and
hands raw pointers to ``xqt_b200_w4a16_run``.
"""

from __future__ import annotations

import torch

from .. import native
from ..errors import XQTBackendError

_GEMV_MAX_M = 16


def _check_cuda(name: str, tensor: torch.Tensor | None, device: torch.device) -> None:
    if tensor is None:
        return
    if not tensor.is_cuda or tensor.device != device:
        raise XQTBackendError(f"B200 W4A16 {name} must be a CUDA tensor on {device}")
    if not tensor.is_contiguous():
        raise XQTBackendError(f"B200 W4A16 {name} must be contiguous")


def select_variant(m: int, n: int, k: int, padded_k: int, group_size: int, activation: str = "none",
                   has_residual: bool = False) -> str:
    code = native.library().xqt_b200_w4a16_select_variant(
        m, n, k, padded_k, group_size, native.ACT[activation], int(has_residual))
    return native.VARIANT_NAMES[code]


def w4a16_linear(
    x: torch.Tensor,
    qweight: torch.Tensor,
    scales: torch.Tensor,
    zero_points: torch.Tensor | None = None,
    bias: torch.Tensor | None = None,
    residual: torch.Tensor | None = None,
    *,
    group_size: int,
    nibble_signed: bool,
    k: int | None = None,
    activation: str = "none",
    variant: str = "auto",
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """``y = x @ dequant(qweight).T (+bias) (+residual)`` with fp32 accumulation.

    x ``[M,K]`` fp16/bf16; qweight ``uint8 [N, padded_K/2]``; scales / zero_points ``[N, G]``
    fp16/bf16/fp32 (same dtype); bias ``[N]`` (converted to fp32); residual ``[M,N]`` of x's dtype.
    """

    if x.ndim != 2 or x.dtype not in (torch.float16, torch.bfloat16):
        raise XQTBackendError("B200 W4A16 activation must be rank-2 fp16/bf16")
    device = x.device
    m, kx = int(x.shape[0]), int(x.shape[1])
    k = kx if k is None else int(k)
    if kx != k:
        raise XQTBackendError("B200 W4A16 activation K disagrees with the weight's logical K")
    if qweight.ndim != 2 or qweight.dtype != torch.uint8:
        raise XQTBackendError("B200 W4A16 qweight must be uint8 [N, padded_K/2]")
    n, padded_k = int(qweight.shape[0]), int(qweight.shape[1]) * 2
    groups = padded_k // int(group_size)
    if scales.dtype not in native.DTYPE_CODE or tuple(scales.shape) != (n, groups):
        raise XQTBackendError(f"B200 W4A16 scales must be [{n},{groups}] fp16/bf16/fp32")
    if zero_points is not None and (zero_points.dtype != scales.dtype or zero_points.shape != scales.shape):
        raise XQTBackendError("B200 W4A16 zero_points must match scales in shape and dtype")
    if activation not in native.ACT:
        raise XQTBackendError(f"B200 W4A16 unknown epilogue activation {activation!r}")
    if bias is not None:
        if bias.numel() != n:
            raise XQTBackendError("B200 W4A16 bias must have N elements")
        bias = bias.reshape(-1).to(device=device, dtype=torch.float32).contiguous()
    if residual is not None and (residual.dtype != x.dtype or tuple(residual.shape) != (m, n)):
        raise XQTBackendError("B200 W4A16 residual must be [M,N] in the activation dtype")
    for name, tensor in (("activation", x), ("qweight", qweight), ("scales", scales),
                         ("zero_points", zero_points), ("residual", residual)):
        _check_cuda(name, tensor, device)
    if out is None:
        out = torch.empty((m, n), device=device, dtype=x.dtype)
    elif out.dtype != x.dtype or tuple(out.shape) != (m, n) or not out.is_contiguous() or out.device != device:
        raise XQTBackendError("B200 W4A16 out must be a contiguous [M,N] tensor in the activation dtype")
    if m == 0:
        return out
    lib = native.library()
    scratch = native.workspace(device, lib.xqt_b200_w4a16_workspace_bytes(m, n, k))
    stream = native.stream_handle(device)
    act_code, param_code = native.DTYPE_CODE[x.dtype], native.DTYPE_CODE[scales.dtype]

    def run(xs, res, dst, rows, which):
        code = lib.xqt_b200_w4a16_run(
            xs.data_ptr(), qweight.data_ptr(), scales.data_ptr(), native.ptr(zero_points), native.ptr(bias),
            native.ptr(res), dst.data_ptr(), rows, n, k, padded_k, int(group_size), int(bool(nibble_signed)),
            act_code, param_code, native.ACT[activation], scratch.data_ptr(), scratch.numel(),
            native.VARIANT[which], stream)
        native.check(code, "xqt_b200_w4a16_run")

    with torch.cuda.device(device):
        run(x, residual, out, m, variant)
    return out


def _fake(x, qweight, scales, zero_points=None, bias=None, residual=None, *, group_size, nibble_signed,
          k=None, activation="none", variant="auto", out=None):
    return x.new_empty((x.shape[0], qweight.shape[0]))


def _register() -> None:
    """Expose the op under xqt's reserved custom-op namespace; harmless if already present."""

    try:
        op = torch.library.custom_op(
            "xqt_operator_opt::b200_w4a16_linear", mutates_args=(), device_types="cuda"
        )(_custom_op_entry)
        op.register_fake(_custom_op_fake)
    except Exception:  # noqa: BLE001 - re-import in one process, or torch without custom_op
        pass


def _custom_op_entry(x: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor,
                     zero_points: torch.Tensor | None, bias: torch.Tensor | None,
                     residual: torch.Tensor | None, group_size: int, nibble_signed: bool,
                     activation: str) -> torch.Tensor:
    return w4a16_linear(x, qweight, scales, zero_points, bias, residual, group_size=group_size,
                        nibble_signed=nibble_signed, activation=activation)


def _custom_op_fake(x, qweight, scales, zero_points, bias, residual, group_size, nibble_signed, activation):
    return x.new_empty((x.shape[0], qweight.shape[0]))


_register()

__all__ = ["select_variant", "w4a16_linear"]
