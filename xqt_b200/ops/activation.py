"""Activation prologue: rotation + dynamic quantisation (one C-ABI call)."""

from __future__ import annotations

import torch

from .. import native
from ..errors import XQTBackendError
from ..quantize import Rotation

_KIND = {None: 0, "regular": 1, "sylvester": 2}
_scale_cache: dict[tuple, torch.Tensor] = {}


def _column_scale(rotation: Rotation, device: torch.device) -> torch.Tensor:
    """The rotation's column factors on ``device``, cached per Rotation object (the entry keeps the object alive, so
    its id cannot be reused; building a key from the sign vector on every call cost more host time than the launch)."""

    key = (id(rotation), device.type, device.index)
    cached = _scale_cache.get(key)
    if cached is None or cached[0] is not rotation:
        cached = (rotation, rotation.column_scale.to(device).contiguous())
        _scale_cache[key] = cached
    return cached[1]


def rotate_quantize(x: torch.Tensor, rotation: Rotation | None, *, bits: int, group_size: int = 64,
                    return_rotated: bool = False, out: tuple | None = None, sign_magnitude: bool = False,
                    tiled_scales: bool = False, scale_in_act_dtype: bool = False):
    """-> (codes int8 ``[M,K]``, scales fp32 ``[M]`` (bits=8) or ``[M, K/group]`` (bits=4)[, rotated x]).

    ``sign_magnitude`` (bits=4 only) writes each int4 code as the byte ``sign << 7 | magnitude`` -- read as
    FP8 E4M3 that is ``code * 2**-9`` exactly, the operand form of the W4A4 GEMM; :func:`decode_sign_magnitude`
    turns such bytes back into two's-complement codes.

    ``tiled_scales`` (with ``sign_magnitude``, group 64 or 0) orders the scales tile-major for the W4A4 GEMM: the
    returned buffer has ``ceil(M/128)*128`` rows of storage and holds ``[ceil(M/128)][K/64][128]``.

    ``scale_in_act_dtype`` (bits=8): the per-token scale is ``T(amax/127)`` rounded to the activation dtype, 0 with
    all-zero codes for an all-zero token -- the SVDQuant W8A8 activation form (gemm_w8a8.cuh:236-262).

    ``out = (codes, scales[, rotated])`` supplies preallocated buffers whose leading ``M`` rows are
    written (a workspace sized for at least M rows): the call then allocates nothing."""

    if x.ndim != 2 or x.dtype not in (torch.float16, torch.bfloat16) or not x.is_cuda:
        raise XQTBackendError("rotate_quantize expects a CUDA rank-2 fp16/bf16 activation")
    if bits not in (4, 8):
        raise XQTBackendError("rotate_quantize supports 8-bit per-token or 4-bit per-group codes")
    if sign_magnitude and bits != 4:
        raise XQTBackendError("sign-magnitude bytes are the form of 4-bit codes only")
    if scale_in_act_dtype and bits != 8:
        raise XQTBackendError("the activation-dtype scale is a form of the 8-bit per-token codes only")
    if tiled_scales and not (sign_magnitude and int(group_size) in (0, 64)):
        raise XQTBackendError("tile-major scales go with sign-magnitude codes of group 64 (or per-token) only")
    x = x.contiguous()
    m, k = int(x.shape[0]), int(x.shape[1])
    device = x.device
    if rotation is not None and k % rotation.block:
        raise XQTBackendError("the rotated dimension must be a multiple of the rotation block")
    per_token4 = bits == 4 and int(group_size) == 0      # one int4 scale per token, replicated per 64-K slot
    if bits == 4 and (k % 64 if per_token4 else k % group_size):
        raise XQTBackendError("K must be a multiple of the activation group size")
    scale_groups = k // 64 if per_token4 else (k // group_size if bits == 4 else 0)
    scale_rows = -(-m // 128) * 128 if tiled_scales else m
    if out is None:
        codes = torch.empty((m, k), device=device, dtype=torch.int8)
        scales = torch.empty((m,) if bits == 8 else (scale_rows, scale_groups), device=device, dtype=torch.float32)
        rotated = torch.empty_like(x) if return_rotated else None
    else:
        codes, scales = out[0][:m], out[1][:scale_rows]
        rotated = out[2][:m] if return_rotated else None
        want_scales = (m,) if bits == 8 else (scale_rows, scale_groups)
        if codes.dtype != torch.int8 or tuple(codes.shape) != (m, k) or not codes.is_contiguous() \
                or scales.dtype != torch.float32 or tuple(scales.shape) != want_scales or not scales.is_contiguous() \
                or (rotated is not None and (rotated.dtype != x.dtype or tuple(rotated.shape) != (m, k) or not rotated.is_contiguous())):
            raise XQTBackendError("rotate_quantize: workspace buffers do not match the activation")
    if m:
        cs = None if rotation is None else _column_scale(rotation, device)
        with torch.cuda.device(device):
            code = native.library().xqt_b200_rotate_quantize(
                x.data_ptr(), native.ptr(cs), codes.data_ptr(), scales.data_ptr(), native.ptr(rotated), m, k,
                _KIND[None if rotation is None else rotation.kind], 0 if rotation is None else rotation.block,
                (6 if tiled_scales else 5) if sign_magnitude else (9 if scale_in_act_dtype else bits), int(group_size), native.DTYPE_CODE[x.dtype], native.stream_handle(device))
        native.check(code, "xqt_b200_rotate_quantize")
    return (codes, scales, rotated) if return_rotated else (codes, scales)


def decode_sign_magnitude(codes: torch.Tensor) -> torch.Tensor:
    """Sign-magnitude code bytes (``sign << 7 | magnitude``) -> two's-complement int8 codes."""

    raw = codes.view(torch.uint8).to(torch.int16)
    magnitude = raw & 0x7F
    return torch.where(raw >= 0x80, -magnitude, magnitude).to(torch.int8)


def quantize_int8_per_tensor(x: torch.Tensor, *, eps: float = 1e-6, out: tuple | None = None):
    """Per-tensor dynamic int8 codes, the activation side of xqt's ``Int8MmaLinear``
    (xqt/contracts/int8_mma.py:135-149,308-319): ``scale = max(absmax, eps)/127``, codes clamped to
    [-127, 127].  -> (codes int8 ``[M,K]``, row_scales fp32 ``[M]`` (the scale, once per row), scale fp32 ``[1]``)."""

    if x.ndim != 2 or x.dtype not in (torch.float16, torch.bfloat16) or not x.is_cuda:
        raise XQTBackendError("quantize_int8_per_tensor expects a CUDA rank-2 fp16/bf16 activation")
    x = x.contiguous()
    m, k = int(x.shape[0]), int(x.shape[1])
    if k % 8:
        raise XQTBackendError("per-tensor int8 quantisation needs K % 8 == 0")
    device = x.device
    if out is None:
        codes = torch.empty((m, k), device=device, dtype=torch.int8)
        rows = torch.empty((m,), device=device, dtype=torch.float32)
        stats = torch.empty((2,), device=device, dtype=torch.float32)
    else:
        codes, rows, stats = out[0][:m], out[1][:m], out[2]
    if m:
        with torch.cuda.device(device):
            code = native.library().xqt_b200_quantize_per_tensor(
                x.data_ptr(), codes.data_ptr(), rows.data_ptr(), stats.data_ptr(), m, k, native.DTYPE_CODE[x.dtype],
                float(eps), native.stream_handle(device))
        native.check(code, "xqt_b200_quantize_per_tensor")
    return codes, rows, stats[1:2]


__all__ = ["decode_sign_magnitude", "quantize_int8_per_tensor", "rotate_quantize"]
