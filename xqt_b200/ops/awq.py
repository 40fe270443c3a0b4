"""AWQ W4A16 decode ops under the names and signatures of xqt's sm_89 backend.

xqt's native decode path is three steps (xqt/kernels/ops/_impl/gemm_backends/sm89/awq_w4a16_decode_sm89.py:16-248,
xqt/kernels/ops/_impl/cuda/awq_w4a16_sm89.py:111-302):

1. ``prepack_sm89_awq_w4a16_decode(weight)``: canonical ``PackedWeight`` -> execution ``PackedWeight``
   (``storage_layout="sm89_awq_w4a16_interleaved_v1"``, ``canonical_qweight`` kept beside it);
2. ``prepare_sm89_awq_w4a16_decode_parameters(weight, spec=, dtype=)`` -> the three immutable tensors
   ``(qweight, scales, scaled_zeros)`` the kernel reads;
3. ``awq_w4a16_decode(inputs, qweight, scales, scaled_zeros, *, output=None)`` or the hot closure
   ``bind_awq_w4a16_decode(qweight, scales, scaled_zeros, *, rows, input_features, output_features,
   dtype, device, bias=None)``.

The functions below are the B200 twins, same order, same argument meaning, same error type.  The
tensor *contents* are backend-private there and here; on B200 they are

* ``qweight``       uint8 ``[tiles, K/128, 4, 2, 2, 32, 16]``: the lane-ordered layout ``b200_w4_lanes_v1``
  (unsigned codes);
* ``scales``        ``[tiles, K/128, 128/g, 4, 8, 4]`` in the dtype of the canonical scales;
* ``scaled_zeros``  zero points in the same order and dtype.  They are NOT pre-multiplied by the scale
  (the sm_89 kernel takes ``-zero * scale`` rounded to fp16/bf16; here the zero point enters an fp32
  fold, which keeps the result equal to the contract reference, xqt/kernels/ops/gemm/reference.py:263-271).

Differences in envelope: group 64 or 128 (sm_89: 64 only), rows 1..16 (sm_89: 1..8), signed weights
are accepted by the prepack (stored as ``code + 8`` with zero point 8, the bridge of
xqt/runtime/modules/awq_w4a16_linear.py:25-71).
"""

from __future__ import annotations

from dataclasses import dataclass
from dataclasses import replace as _dc_replace
from typing import Callable

import torch

from .. import native, prepack
from ..contracts import PackedWeight, PackedWeightMetadata
from ..errors import NativeLibraryError, XQTBackendError
from ..layout import W4_LAYOUT, validate_w4a16_packed_weight
from ..weakid import WeakIdDict

LANES_LAYOUT = "b200_w4_lanes_v1"
LANES_PACK_VERSION = "xqt-b200-awq-w4a16-v1"
_SUPPORTED_DTYPES = (torch.float16, torch.bfloat16)


def native_awq_w4a16_available(*, build: bool = False) -> bool:
    """Whether the B200 decode backend can run on the current device (cf. awq_w4a16_sm89.py:111-130).
    ``build=True`` additionally loads the shared library (nothing is compiled at run time here)."""

    import os

    if not torch.cuda.is_available() or torch.cuda.get_device_capability() != (10, 0):
        return False
    if os.environ.get("XQT_DISABLE_B200", "0") not in {"", "0"}:
        return False
    if not build:
        return native.LIBRARY_PATH.exists()
    return native.available()


def native_awq_w4a16_shape_supported(rows: int, input_features: int, output_features: int, group_size: int = 128) -> bool:
    try:
        lib = native.library()
    except NativeLibraryError:
        return False
    return bool(lib.xqt_b200_w4a16_decode_lanes_supported(int(rows), int(output_features), int(input_features), int(group_size)))


def native_awq_w4a16_version() -> str:
    return native.version()


def prepack_b200_awq_w4a16_decode(weight: PackedWeight) -> PackedWeight:
    """Canonical ``xqt_int4_nk_v1`` weight (CUDA-resident) -> execution ``PackedWeight`` whose ``qweight`` is
    the lane-ordered layout; scales, zero points and the canonical bytes ride along unchanged."""

    if not hasattr(weight, "metadata") or not hasattr(weight, "qweight"):
        raise XQTBackendError("B200 AWQ decode prepack requires a PackedWeight")
    meta = weight.metadata
    if meta.weight_dtype != "int4" or meta.storage_layout != W4_LAYOUT or meta.group_size not in (64, 128):
        raise XQTBackendError("B200 AWQ decode prepack requires canonical INT4 with group_size 64 or 128")
    n, k = (int(v) for v in meta.logical_shape)
    if int(meta.padded_k) != k or k % 128:
        raise XQTBackendError("B200 AWQ decode prepack requires K == padded_K and K % 128 == 0")
    qweight = weight.qweight
    if not isinstance(qweight, torch.Tensor) or qweight.dtype != torch.uint8 or tuple(qweight.shape) != (n, k // 2):
        raise XQTBackendError("canonical AWQ qweight must be uint8 [N,K/2]")
    if not qweight.is_cuda:
        raise XQTBackendError("B200 AWQ decode prepack requires CUDA-resident weights")
    scales, zeros = weight.scales, weight.zero_points
    if scales is None:
        raise XQTBackendError("B200 AWQ decode prepack requires group scales")
    if zeros is not None and zeros.dtype != scales.dtype:
        zeros = zeros.to(scales.dtype)
    if meta.nibble_signed and zeros is not None:
        raise XQTBackendError("signed INT4 storage carries no zero points")
    tiled = prepack.lanes_w4(qweight.contiguous(), scales.contiguous(), None if zeros is None else zeros.contiguous(),
                             group_size=int(meta.group_size), nibble_signed=bool(meta.nibble_signed), k=k)
    values = {f: getattr(meta, f) for f in PackedWeightMetadata.__dataclass_fields__}
    values.update(storage_layout=LANES_LAYOUT, pack_version=LANES_PACK_VERSION, nibble_signed=False)
    execution = PackedWeight(qweight=tiled.weights, scales=weight.scales, zero_points=weight.zero_points,
                             metadata=PackedWeightMetadata(**values), canonical_qweight=qweight)
    # the lane-ordered parameters ride beside the execution weight, keyed weakly on its qweight tensor
    # (the frozen PackedWeight has no field for them); the record dies with that tensor
    _LANES[tiled.weights] = _LaneRecord(params=tiled.params, nibble_signed=tiled.nibble_signed,
                                        has_zero_point=tiled.has_zero_point)
    return execution


@dataclass(frozen=True)
class _LaneRecord:
    params: torch.Tensor
    nibble_signed: bool
    has_zero_point: bool


_LANES = WeakIdDict()


def _tiled_of(weight: PackedWeight) -> _LaneRecord:
    record = _LANES.get(weight.qweight) if isinstance(weight.qweight, torch.Tensor) else None
    if record is None:
        raise XQTBackendError("B200 AWQ decode requires prepack_b200_awq_w4a16_decode()")
    return record


def prepare_b200_awq_w4a16_decode_parameters(weight: PackedWeight, *, spec=None, dtype: torch.dtype) -> tuple[
        torch.Tensor, torch.Tensor, torch.Tensor | None]:
    """-> ``(qweight, scales, scaled_zeros)`` for :func:`awq_w4a16_decode` / :func:`bind_awq_w4a16_decode`;
    immutable, made once outside the hot path (cf. awq_w4a16_decode_sm89.py:107-128)."""

    if dtype not in _SUPPORTED_DTYPES:
        raise XQTBackendError("B200 AWQ prepared parameters require FP16 or BF16")
    if weight.metadata.storage_layout != LANES_LAYOUT:
        raise XQTBackendError("B200 AWQ decode requires prepack_b200_awq_w4a16_decode()")
    tiled = _tiled_of(weight)
    if spec is not None:
        canonical = _dc_replace(weight, qweight=weight.canonical_qweight, canonical_qweight=None,
                                metadata=_dc_replace(weight.metadata, storage_layout=W4_LAYOUT,
                                                     nibble_signed=tiled.nibble_signed))
        try:
            validate_w4a16_packed_weight(canonical, spec=spec.quant, logical_shape=(spec.problem.n, spec.problem.k))
        except (TypeError, ValueError) as exc:
            raise XQTBackendError(f"B200 AWQ decode: packed weight rejected: {exc}") from exc
    scales = tiled.params[0]
    if tiled.nibble_signed:          # codes were stored + 8: the bridge's zero point
        zeros = torch.full_like(scales, 8.0)
    else:
        zeros = tiled.params[1] if tiled.has_zero_point else None
    return weight.qweight, scales, zeros


def _check_static(qweight, scales, scaled_zeros, *, input_features: int, output_features: int, device: torch.device):
    if qweight.ndim != 7 or qweight.dtype != torch.uint8 or tuple(qweight.shape[2:]) != (4, 2, 2, 32, 16):
        raise XQTBackendError("bound AWQ W4A16 qweight does not match the static execution contract")
    tiles, kblocks = int(qweight.shape[0]), int(qweight.shape[1])
    if kblocks * 128 != input_features or tiles != -(-output_features // 128):
        raise XQTBackendError("bound AWQ W4A16 qweight does not match the static execution contract")
    if scales.ndim != 6 or tuple(scales.shape[:2]) != (tiles, kblocks) or tuple(scales.shape[3:]) != (4, 8, 4) \
            or int(scales.shape[2]) not in (1, 2) or scales.dtype not in native.DTYPE_CODE:
        raise XQTBackendError("bound AWQ W4A16 scales does not match the static execution contract")
    if scaled_zeros is not None and (scaled_zeros.shape != scales.shape or scaled_zeros.dtype != scales.dtype):
        raise XQTBackendError("bound AWQ W4A16 scaled_zeros does not match the static execution contract")
    for name, tensor in (("qweight", qweight), ("scales", scales), ("scaled_zeros", scaled_zeros)):
        if tensor is not None and (tensor.device != device or not tensor.is_contiguous()):
            raise XQTBackendError(f"bound AWQ W4A16 {name} does not match the static execution contract")
    return 128 // int(scales.shape[2])


def bind_awq_w4a16_decode(qweight: torch.Tensor, scales: torch.Tensor, scaled_zeros: torch.Tensor | None, *, rows: int,
                          input_features: int, output_features: int, dtype: torch.dtype, device: torch.device,
                          bias: torch.Tensor | None = None) -> Callable[[torch.Tensor], torch.Tensor]:
    """Bind the immutable execution tensors to the C-ABI entry (cf. awq_w4a16_sm89.py:217-302).  Static
    tensors are validated here; the returned callable assumes its input already is ``[rows, input_features]``
    in ``dtype`` on ``device`` and makes one library call."""

    rows, input_features, output_features = int(rows), int(input_features), int(output_features)
    device = torch.device(device)
    if not 1 <= rows <= 16:
        raise XQTBackendError("bound AWQ W4A16 decode requires 1 <= rows <= 16")
    if dtype not in _SUPPORTED_DTYPES:
        raise XQTBackendError("bound AWQ W4A16 decode requires FP16 or BF16")
    if device.type != "cuda":
        raise XQTBackendError("bound AWQ W4A16 decode requires a CUDA device")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    group = _check_static(qweight, scales, scaled_zeros, input_features=input_features, output_features=output_features,
                          device=device)
    lib = native.library()
    if not lib.xqt_b200_w4a16_decode_lanes_supported(rows, output_features, input_features, group):
        raise XQTBackendError("bound AWQ W4A16 decode: shape outside the B200 kernel's envelope")
    bias32 = None
    if bias is not None:
        if bias.device != device or tuple(bias.shape) != (output_features,):
            raise XQTBackendError("bound AWQ W4A16 bias does not match the static execution contract")
        bias32 = bias.to(torch.float32).contiguous()
    fn = lib.xqt_b200_w4a16_decode_lanes
    status = native.status_word(device)
    args_head = (qweight.data_ptr(), scales.data_ptr(), native.ptr(scaled_zeros), native.ptr(bias32), 0)
    args_tail = (rows, output_features, input_features, group, 0, native.DTYPE_CODE[dtype], native.DTYPE_CODE[scales.dtype],
                 native.DTYPE_CODE[dtype], 0, status.data_ptr())

    def bound(inputs: torch.Tensor) -> torch.Tensor:
        output = torch.empty((rows, output_features), dtype=dtype, device=device)
        code = fn(inputs.data_ptr(), *args_head, output.data_ptr(), *args_tail, torch.cuda.current_stream(device).cuda_stream)
        if code != 0:
            native.check(code, "xqt_b200_w4a16_decode_lanes")
        return output

    bound.keep = (qweight, scales, scaled_zeros, bias32, status)     # the raw pointers above must stay valid
    return bound


def awq_w4a16_decode(inputs: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor,
                     scaled_zeros: torch.Tensor | None, *, output: torch.Tensor | None = None) -> torch.Tensor:
    """One ``M <= 16`` decode projection (cf. awq_w4a16_sm89.py:152-179).  The output width is taken from
    ``output`` when given, else it is ``128 * tiles`` (layers whose N is not a multiple of 128 pass ``output``
    or use :func:`bind_awq_w4a16_decode`)."""

    return awq_w4a16_decode_bias(inputs, qweight, scales, scaled_zeros, None, output=output)


def awq_w4a16_decode_bias(inputs: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor,
                          scaled_zeros: torch.Tensor | None, bias: torch.Tensor | None, *,
                          output: torch.Tensor | None = None) -> torch.Tensor:
    """Decode with a fused output bias (cf. awq_w4a16_sm89.py:182-214)."""

    if inputs.ndim != 2 or inputs.dtype not in _SUPPORTED_DTYPES:
        raise XQTBackendError("AWQ W4A16 inputs must be FP16/BF16 rank-2")
    if not inputs.is_cuda:
        raise XQTBackendError("AWQ W4A16 inputs must be CUDA")
    rows, k = int(inputs.shape[0]), int(inputs.shape[1])
    n = int(qweight.shape[0]) * 128 if output is None else int(output.shape[1])
    run = bind_awq_w4a16_decode(qweight, scales, scaled_zeros, rows=rows, input_features=k, output_features=n,
                                dtype=inputs.dtype, device=inputs.device, bias=bias)
    result = run(inputs.contiguous())
    if output is None:
        return result
    if output.dtype != inputs.dtype or tuple(output.shape) != (rows, n):
        raise XQTBackendError("AWQ W4A16 output must be [rows, output_features] in the input dtype")
    output.copy_(result)
    return output


def bind_awq_w4a8_decode(qweight: torch.Tensor, scales: torch.Tensor, scaled_zeros: torch.Tensor | None, *, rows: int,
                         input_features: int, output_features: int, dtype: torch.dtype, device: torch.device,
                         residual: bool = False) -> Callable:
    """W4A8 decode: int8 activation codes with ONE activation scale against the same W4 execution layout,
    ``y = s_a * sum_g s_w[n,g] * sum_{k in g} a_q[m,k] (code[n,k] - zero[n,g])`` (cf. ``bind_awq_w4a8_decode`` and the
    DP4A kernel it binds, awq_w4a16_sm89.py:386-430, awq_w4a16_sm89_kernel.cu:595-724).  On B200 the integer codes go
    through the cluster decode kernel as exact bf16/fp16 integers (|a_q| <= 127 is exact in either format, a group's
    integer sum stays below 2^24), fp32 sums out, and the activation scale and rounding are one elementwise pass.
    ``dtype`` is the output dtype (the reference takes it from ``scales``).  Returns ``run(codes, scale_a[, residual])``;
    with ``residual=True`` the residual row is added in the output dtype, as the reference's ``_bias`` form does."""

    rows, input_features, output_features = int(rows), int(input_features), int(output_features)
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    if not 1 <= rows <= 16 or dtype not in _SUPPORTED_DTYPES or device.type != "cuda":
        raise XQTBackendError("bound AWQ W4A8 decode requires 1 <= rows <= 16, an FP16/BF16 output dtype and a CUDA device")
    group = _check_static(qweight, scales, scaled_zeros, input_features=input_features, output_features=output_features,
                          device=device)
    lib = native.library()
    if not lib.xqt_b200_w4a16_decode_lanes_supported(rows, output_features, input_features, group):
        raise XQTBackendError("bound AWQ W4A8 decode: shape outside the B200 kernel's envelope")
    fn = lib.xqt_b200_w4a16_decode_lanes
    status = native.status_word(device)
    head = (qweight.data_ptr(), scales.data_ptr(), native.ptr(scaled_zeros), 0, 0)
    tail = (rows, output_features, input_features, group, 0, native.DTYPE_CODE[dtype], native.DTYPE_CODE[scales.dtype],
            native.DTYPE_CODE[torch.float32], 0, status.data_ptr())
    sums = torch.empty((rows, output_features), dtype=torch.float32, device=device)

    def bound(codes: torch.Tensor, scale_a, residual_row: torch.Tensor | None = None) -> torch.Tensor:
        if codes.dtype != torch.int8 or tuple(codes.shape) != (rows, input_features) or codes.device != device:
            raise XQTBackendError("AWQ W4A8 inputs must be INT8 [rows, input_features] on the bound device")
        exact = codes.to(dtype)                                       # integers up to 127: exact in fp16 and bf16
        code = fn(exact.data_ptr(), *head, sums.data_ptr(), *tail, torch.cuda.current_stream(device).cuda_stream)
        if code != 0:
            native.check(code, "xqt_b200_w4a16_decode_lanes")
        scale = scale_a.to(device=device, dtype=torch.float32).reshape(()) if isinstance(scale_a, torch.Tensor) else float(scale_a)
        out = (sums * scale).to(dtype)
        if residual:
            if residual_row is None or residual_row.dtype != dtype or tuple(residual_row.shape) != (rows, output_features):
                raise XQTBackendError("AWQ W4A8 residual must be [rows, output_features] in the output dtype")
            out = out + residual_row
        return out

    bound.keep = (qweight, scales, scaled_zeros, status, sums)
    return bound


def awq_w4a8_decode(inputs: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor, scale_a, *,
                    scaled_zeros: torch.Tensor | None = None, dtype: torch.dtype | None = None,
                    output: torch.Tensor | None = None) -> torch.Tensor:
    """One W4A8 decode projection (cf. awq_w4a16_sm89.py:305-341): ``inputs`` int8 ``[M <= 16, K]``, ``scale_a`` a
    tensor or a float.  ``scaled_zeros`` is the zero-point plane of the execution layout (None: symmetric, stored as
    ``code ^ 8``); the output dtype is ``dtype``, by default the dtype of ``scales`` when that is fp16 / bf16, else bf16."""

    if inputs.ndim != 2 or inputs.dtype != torch.int8:
        raise XQTBackendError("AWQ W4A8 inputs must be INT8 rank-2")
    if not inputs.is_cuda:
        raise XQTBackendError("AWQ W4A8 inputs must be CUDA")
    odt = dtype if dtype is not None else (scales.dtype if scales.dtype in _SUPPORTED_DTYPES else torch.bfloat16)
    rows, k = int(inputs.shape[0]), int(inputs.shape[1])
    n = int(qweight.shape[0]) * 128 if output is None else int(output.shape[1])
    run = bind_awq_w4a8_decode(qweight, scales, scaled_zeros, rows=rows, input_features=k, output_features=n, dtype=odt,
                               device=inputs.device)
    result = run(inputs.contiguous(), scale_a)
    if output is None:
        return result
    output.copy_(result)
    return output


def b200_awq_w4a16_decode_executor(activation, weight, *, spec, weight_scales=None, activation_scales=None,
                                   weight_zero_points=None, activation_zero_points=None, bias=None, residual=None,
                                   **_unused) -> torch.Tensor:
    """GEMM-registry executor over a weight prepacked by :func:`prepack_b200_awq_w4a16_decode`
    (cf. ``sm89_awq_w4a16_decode_executor``, awq_w4a16_decode_sm89.py:131-248)."""

    if activation_scales is not None or activation_zero_points is not None:
        raise XQTBackendError("W4A16 does not accept activation quantization scales")
    if residual is not None or spec.epilogue.has_residual or spec.epilogue.activation != "none":
        raise XQTBackendError("B200 AWQ decode executor supports an optional bias only")
    if not isinstance(activation, torch.Tensor) or activation.ndim != 2 or not activation.is_cuda:
        raise XQTBackendError("B200 AWQ decode activation must be CUDA rank-2")
    if activation.dtype not in _SUPPORTED_DTYPES or tuple(activation.shape) != (spec.problem.m, spec.problem.k):
        raise XQTBackendError("B200 AWQ decode activation does not match the GemmProblem")
    if not 1 <= spec.problem.m <= 16:
        raise XQTBackendError("B200 AWQ decode requires 1 <= M <= 16")
    qweight, scales, zeros = prepare_b200_awq_w4a16_decode_parameters(weight, spec=spec, dtype=activation.dtype)
    return awq_w4a16_decode_bias(activation, qweight, scales, zeros, bias,
                                 output=torch.empty((spec.problem.m, spec.problem.n), dtype=activation.dtype, device=activation.device))


__all__ = [
    "LANES_LAYOUT", "awq_w4a8_decode", "bind_awq_w4a8_decode", "awq_w4a16_decode", "awq_w4a16_decode_bias", "b200_awq_w4a16_decode_executor", "bind_awq_w4a16_decode",
    "native_awq_w4a16_available", "native_awq_w4a16_shape_supported", "native_awq_w4a16_version",
    "prepack_b200_awq_w4a16_decode", "prepare_b200_awq_w4a16_decode_parameters",
]
