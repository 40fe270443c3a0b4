"""GEMM-registry executors backed by the sm_100a kernels, and their installer.

An executor has xqt's executor signature (xqt/kernels/ops/gemm/dispatch.py:239-250):
``executor(activation, weight, *, spec, weight_scales, activation_scales, weight_zero_points,
activation_zero_points, bias, residual, **kwargs) -> Tensor``; it allocates and returns the
output on ``activation.device``, never mutates its inputs, enqueues on torch's current stream and
raises ``XQTBackendError`` for anything outside its envelope (same checks, same wording pattern,
as ``sm89_w4a16_dequant_executor``, _impl/gemm_backends/sm89/w4a16_sm89.py:198-300).  Only
attributes are read from ``weight`` / ``spec``, so xqt's own ``PackedWeight`` / ``GemmSpec``
objects work as well as this package's mirrors; ``install_b200_executors`` therefore also accepts
xqt's ``GemmKernelRegistry`` (anything with ``register/replace/get``).
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from dataclasses import fields as _dc_fields
from dataclasses import replace as _dc_replace
from typing import Any

import torch

from . import native
from .errors import XQTBackendError
from .layout import validate_w4a16_packed_weight
from .weakid import WeakIdDict
from .registry import B200_SVD_W4A4, B200_W4A16, B200_W8A8, GemmKernelRegistry, b200_rows

_TORCH = {"fp16": torch.float16, "bf16": torch.bfloat16}


def _require_b200(device: torch.device) -> None:
    if os.environ.get("XQT_DISABLE_B200", "") not in {"", "0"}:
        raise XQTBackendError("B200 backend disabled by XQT_DISABLE_B200")
    if device.type != "cuda":
        raise XQTBackendError("B200 executors need CUDA tensors")
    major, minor = torch.cuda.get_device_capability(device)
    if (major, minor) != (10, 0):
        raise XQTBackendError(f"B200 executor received sm_{major}{minor}")


# Decode execution layouts derived from canonical weights, one per weight tensor.  Keyed on the
# tensor object itself (weakly: the entry dies with the weight, so a recycled address can never hit a
# stale layout) and checked against the tensor's version counter, the way xqt's runtime modules key
# their prepacked W4A4 state on data_ptr/_version (xqt/runtime/modules/composite_add_w4a4.py:164-187).
_decode_layouts = WeakIdDict()


def _decode_entry(weight) -> dict | None:
    """The cached decode layout of ``weight`` (built on first use), or None when the layer is outside
    the decode kernel's envelope or XQT_B200_DECODE_PREPACK=0 asks to keep only the canonical bytes."""

    from .ops.w4a16 import prepare_decode

    if os.environ.get("XQT_B200_DECODE_PREPACK", "1") in {"0", ""}:
        return None
    meta = weight.metadata
    group, k = int(meta.group_size), int(meta.logical_shape[1])
    if group not in (64, 128) or int(meta.padded_k) != k or k % 128:
        return None
    qweight, scales, zeros = weight.qweight, weight.scales, weight.zero_points
    versions = (qweight._version, scales._version, None if zeros is None else zeros._version,
                scales.data_ptr(), None if zeros is None else zeros.data_ptr())
    entry = _decode_layouts.get(qweight)
    if entry is None or entry["versions"] != versions:
        if zeros is not None and zeros.dtype != scales.dtype:
            zeros = zeros.to(scales.dtype)
        tiled = prepare_decode(qweight, scales.contiguous(), None if zeros is None else zeros.contiguous(),
                               group_size=group, nibble_signed=bool(meta.nibble_signed), k=k, layout="lanes")
        entry = {"versions": versions, "tiled": tiled, "bound": {}}
        _decode_layouts[qweight] = entry
    return entry


def b200_w4a16_executor(activation, weight, *, spec, weight_scales=None, activation_scales=None,
                        weight_zero_points=None, activation_zero_points=None, bias=None, residual=None,
                        variant: str = "auto", output: torch.Tensor | None = None) -> torch.Tensor:
    """W4A16 on the canonical ``xqt_int4_nk_v1`` PackedWeight, fp16 or bf16, any M."""

    from .ops.w4a16 import w4a16_linear

    if not hasattr(weight, "metadata"):
        raise XQTBackendError("B200 W4A16 requires a canonical PackedWeight")
    quant, problem = spec.quant, spec.problem
    if quant.activation_dtype not in _TORCH:
        raise XQTBackendError("B200 W4A16 supports fp16 or bf16 activations")
    if quant.output_dtype != quant.activation_dtype:
        raise XQTBackendError("B200 W4A16 requires output dtype equal to activation dtype")
    if activation_scales is not None or activation_zero_points is not None:
        raise XQTBackendError("W4A16 does not accept activation quantization scales")
    try:
        validate_w4a16_packed_weight(weight, spec=quant, logical_shape=(problem.n, problem.k))
    except (TypeError, ValueError) as exc:
        raise XQTBackendError(f"B200 W4A16 packed weight rejected: {exc}") from exc
    if weight_scales is not None and weight_scales is not weight.scales and not torch.equal(weight_scales, weight.scales):
        raise XQTBackendError("external weight_scales disagree with PackedWeight.scales")
    if (weight_zero_points is not None and weight_zero_points is not weight.zero_points
            and not torch.equal(weight_zero_points, weight.zero_points)):
        raise XQTBackendError("external weight_zero_points disagree with PackedWeight.zero_points")
    if not isinstance(activation, torch.Tensor) or activation.ndim != 2 or not activation.is_cuda:
        raise XQTBackendError("B200 W4A16 activation must be CUDA rank-2")
    _require_b200(activation.device)
    if activation.dtype != _TORCH[quant.activation_dtype]:
        raise XQTBackendError("B200 W4A16 activation dtype disagrees with QuantSpec")
    if tuple(activation.shape) != (problem.m, problem.k):
        raise XQTBackendError("B200 W4A16 activation shape does not match GemmProblem")
    if spec.epilogue.has_bias and bias is None:
        raise XQTBackendError("W4A16 epilogue declares bias but no bias was supplied")
    if spec.epilogue.has_residual and residual is None:
        raise XQTBackendError("W4A16 epilogue declares residual but no residual was supplied")
    if bias is not None and tuple(bias.shape) not in {(problem.n,), (1, problem.n)}:
        raise XQTBackendError("B200 W4A16 bias must have shape [N] or [1,N]")
    # decode sizes: the cluster split-K kernel on the lane-ordered layout derived (once) from this weight
    if (variant == "auto" and 1 <= problem.m <= 16 and spec.epilogue.activation == "none"
            and native.library().xqt_b200_w4a16_decode_lanes_supported(
                problem.m, problem.n, problem.k, int(weight.metadata.group_size))):
        entry = _decode_entry(weight)
        if entry is not None:
            from .ops.w4a16 import bind_w4a16_decode

            # one bound callable per (rows, dtype) and bias tensor; the bias is a weak key too
            slot = entry["bound"].setdefault((problem.m, activation.dtype), {"plain": None, "biased": WeakIdDict()})
            if bias is None:
                run = slot["plain"]
            else:
                hit = slot["biased"].get(bias)
                run = hit[1] if hit is not None and hit[0] == bias._version else None
            if run is None:
                run = bind_w4a16_decode(entry["tiled"], rows=problem.m, dtype=activation.dtype, bias=bias)
                if bias is None:
                    slot["plain"] = run
                else:
                    slot["biased"][bias] = (bias._version, run)
            return run(activation.contiguous(), output, None if residual is None else residual.contiguous())
    scales, zeros = weight.scales, weight.zero_points
    if zeros is not None and zeros.dtype != scales.dtype:
        zeros = zeros.to(scales.dtype)
    return w4a16_linear(
        activation.contiguous(), weight.qweight, scales.contiguous(), None if zeros is None else zeros.contiguous(),
        bias, None if residual is None else residual.contiguous(), group_size=int(weight.metadata.group_size),
        nibble_signed=bool(weight.metadata.nibble_signed), k=problem.k, activation=spec.epilogue.activation,
        variant=variant, out=output,
    )


def b200_w8a8_executor(activation, weight, *, spec, weight_scales=None, activation_scales=None,
                       weight_zero_points=None, activation_zero_points=None, bias=None, residual=None,
                       output: torch.Tensor | None = None) -> torch.Tensor:
    """W8A8 of the GEMM contract (xqt/kernels/ops/gemm/reference.py:278-323, quantize.py:60-131):
    ``weight`` int8 ``[N, K]`` with per-output-channel ``weight_scales [N]``; ``activation`` either
    int8 ``[M, K]`` with per-token ``activation_scales`` (``[M]`` or ``[M,1]``) or fp16/bf16, which is
    quantised per token here (``amax/127``, clamp [-128,127]) by the prologue kernel.  Output in
    ``QuantSpec.output_dtype`` (fp16 / bf16): ``acc * a_scale[m] * w_scale[n] (+ bias)``."""

    from .ops.activation import rotate_quantize
    from .ops.w8a8 import PackedConvRotW8A8Linear, w8a8_gemm

    quant, problem = spec.quant, spec.problem
    if quant.weight_dtype != "int8" or quant.activation_dtype != "int8":
        raise XQTBackendError("B200 W8A8 executor serves int8 weights with int8 activations")
    if quant.output_dtype not in _TORCH:
        raise XQTBackendError("B200 W8A8 output dtype must be fp16 or bf16")
    if quant.weight_granularity != "per_channel" or quant.activation_granularity not in ("per_token", "per_tensor"):
        raise XQTBackendError("B200 W8A8 supports per-channel weight scales with per-token or per-tensor activation scales")
    per_tensor = quant.activation_granularity == "per_tensor"
    if weight_zero_points is not None or activation_zero_points is not None or quant.activation_zero_point:
        raise XQTBackendError("B200 W8A8 is symmetric: zero points are not supported")
    if residual is not None or spec.epilogue.has_residual or spec.epilogue.activation != "none":
        raise XQTBackendError("B200 W8A8 epilogue supports bias only")
    qweight = getattr(weight, "qweight", weight)
    if weight_scales is None:
        weight_scales = getattr(weight, "scales", None)
    if not isinstance(qweight, torch.Tensor) or qweight.dtype != torch.int8 or tuple(qweight.shape) != (problem.n, problem.k):
        raise XQTBackendError("B200 W8A8 weight must be int8 [N, K]")
    if weight_scales is None or weight_scales.numel() != problem.n:
        raise XQTBackendError("B200 W8A8 needs per-channel weight_scales with N entries")
    if not isinstance(activation, torch.Tensor) or activation.ndim != 2 or not activation.is_cuda:
        raise XQTBackendError("B200 W8A8 activation must be CUDA rank-2")
    _require_b200(activation.device)
    if tuple(activation.shape) != (problem.m, problem.k):
        raise XQTBackendError("B200 W8A8 activation shape does not match GemmProblem")
    if problem.k % 16 or problem.n % 8:
        raise XQTBackendError("B200 W8A8 needs K % 16 == 0 and N % 8 == 0")
    device, dtype = activation.device, _TORCH[quant.output_dtype]
    if activation.dtype == torch.int8:
        want = 1 if per_tensor else problem.m
        if activation_scales is None or activation_scales.numel() != want:
            raise XQTBackendError(f"int8 activations need activation_scales with {want} entries")
        codes = activation.contiguous()
        a_scale = activation_scales.reshape(-1).to(device=device, dtype=torch.float32)
        a_scale = (a_scale.expand(problem.m) if per_tensor else a_scale).contiguous()
    elif activation.dtype in (torch.float16, torch.bfloat16):
        if activation_scales is not None:
            raise XQTBackendError("floating activations are quantised dynamically: do not pass activation_scales")
        if per_tensor:
            # Int8MmaLinear semantics (xqt/contracts/int8_mma.py:135-149,317-319): one scale, clamp +-127
            from .ops.activation import quantize_int8_per_tensor

            codes, a_scale, _ = quantize_int8_per_tensor(activation.contiguous())
        else:
            codes, a_scale = rotate_quantize(activation.contiguous(), None, bits=8)
    else:
        raise XQTBackendError("B200 W8A8 activation must be int8, fp16 or bf16")
    packed = PackedConvRotW8A8Linear(
        qweight=qweight.to(device).contiguous(),
        weight_scales=weight_scales.reshape(-1).to(device=device, dtype=torch.float32).contiguous(),
        bias=None if bias is None else bias.reshape(-1).to(device=device, dtype=torch.float32).contiguous(),
        input_features=problem.k, output_features=problem.n, padded_input_features=problem.k, dtype=dtype)
    return w8a8_gemm(codes, a_scale, packed, output)


@dataclass(frozen=True, slots=True)
class SVDGemmContract:
    """GEMM-side description of "quantised main + low-rank correction" (fields and checks of xqt's
    ``SVDGemmContract``, xqt/kernels/ops/gemm/p4.py:612-640).  ``fusion_boundary`` says where a backend
    may merge the low-rank branch into the main GEMM; the B200 kernel computes the down projection in
    its own pass and fuses the up projection into the epilogue, i.e. it implements ``fuse_up`` and
    accepts the other two values as requests it over-satisfies."""

    main_spec: Any
    rank: int
    outlier_channels: tuple[int, ...] = ()
    fusion_boundary: str = "separate_gemm"
    outlier_mode: str = "correction"

    def __post_init__(self) -> None:
        if int(self.rank) < 1:
            raise ValueError("SVD rank must be positive")
        if self.fusion_boundary not in ("separate_gemm", "fuse_down", "fuse_up"):
            raise ValueError("unsupported SVD fusion_boundary")
        if self.outlier_mode not in ("correction", "replacement"):
            raise ValueError("unsupported SVD outlier_mode")
        channels = tuple(int(c) for c in self.outlier_channels)
        k = int(self.main_spec.problem.k)
        if len(set(channels)) != len(channels) or any(not 0 <= c < k for c in channels):
            raise ValueError("SVD outlier_channels must be unique valid K indices")
        object.__setattr__(self, "outlier_channels", channels)

    def to_dict(self) -> dict[str, Any]:
        return {"main_spec": self.main_spec.to_dict(), "rank": int(self.rank), "outlier_channels": list(self.outlier_channels),
                "fusion_boundary": self.fusion_boundary, "outlier_mode": self.outlier_mode}


_svd_layers = WeakIdDict()      # residual qweight tensor -> (identity of the other tensors, packed layer)


def b200_svd_w4a4_executor(activation, weight, *, spec, weight_scales=None, activation_scales=None,
                           weight_zero_points=None, activation_zero_points=None, bias=None, residual=None,
                           low_rank_down: torch.Tensor | None = None, low_rank_up: torch.Tensor | None = None,
                           contract: SVDGemmContract | None = None, rotation=None,
                           output: torch.Tensor | None = None) -> torch.Tensor:
    """SVDQuant dual path behind the GEMM registry: ``weight`` is the int4 residual as a canonical signed
    ``xqt_int4_nk_v1`` PackedWeight with group-64 scales (the composite artifact's ``packed_residual`` /
    ``residual_scale``, xqt/contracts/composite.py:92-227), ``low_rank_down [r,K]`` / ``low_rank_up [N,r]``
    the rank-r pair.  The activation (fp16 / bf16, already rotated unless ``rotation`` is given) is
    quantised to int4 per (token, 64-K) inside the call, as xqt's native W4A4 path does
    (xqt/kernels/ops/_impl/cute/svdq_w4a4_sm89.py:1203-1262); the sum is what ``reference_svd_dual_path``
    computes (p4.py:687-767) up to that activation rounding."""

    from .ops.w4a4 import GROUP, pack_svdq_w4a4_linear, svdq_w4a4_linear

    if low_rank_down is None or low_rank_up is None:
        raise XQTBackendError("B200 SVD W4A4 needs low_rank_down [r,K] and low_rank_up [N,r]")
    if not hasattr(weight, "metadata"):
        raise XQTBackendError("B200 SVD W4A4 requires the residual as a canonical PackedWeight")
    quant, problem, meta = spec.quant, spec.problem, weight.metadata
    if quant.weight_dtype != "int4" or quant.activation_dtype not in _TORCH or quant.output_dtype != quant.activation_dtype:
        raise XQTBackendError("B200 SVD W4A4 serves int4 weights with fp16/bf16 activations and outputs")
    if not meta.nibble_signed or int(meta.group_size) != GROUP or weight.zero_points is not None:
        raise XQTBackendError("B200 SVD W4A4 needs a symmetric signed residual with group size 64")
    if activation_scales is not None or activation_zero_points is not None or weight_zero_points is not None:
        raise XQTBackendError("B200 SVD W4A4 quantises activations itself and takes no zero points")
    if residual is not None or spec.epilogue.has_residual or spec.epilogue.activation != "none":
        raise XQTBackendError("B200 SVD W4A4 epilogue supports bias only")
    if not isinstance(activation, torch.Tensor) or activation.ndim != 2 or not activation.is_cuda:
        raise XQTBackendError("B200 SVD W4A4 activation must be CUDA rank-2")
    _require_b200(activation.device)
    if activation.dtype != _TORCH[quant.activation_dtype] or tuple(activation.shape) != (problem.m, problem.k):
        raise XQTBackendError("B200 SVD W4A4 activation does not match the GemmProblem / QuantSpec")
    rank = int(low_rank_down.shape[0])
    if tuple(low_rank_down.shape) != (rank, problem.k) or tuple(low_rank_up.shape) != (problem.n, rank):
        raise XQTBackendError("low_rank_down must be [rank,K] and low_rank_up [N,rank]")
    if contract is not None:
        if int(contract.rank) != rank:
            raise XQTBackendError("SVDGemmContract.rank disagrees with the low-rank factors")
        if contract.outlier_channels:
            raise XQTBackendError("B200 SVD W4A4 does not serve outlier-channel corrections")
    scales = weight.scales if weight_scales is None else weight_scales
    if scales is None or tuple(scales.shape) != (problem.n, problem.k // GROUP):
        raise XQTBackendError("B200 SVD W4A4 needs residual scales [N, K/64]")
    identity = (id(scales), scales._version, id(low_rank_down), low_rank_down._version, id(low_rank_up),
                low_rank_up._version, None if bias is None else (id(bias), bias._version), activation.dtype, id(rotation))
    hit = _svd_layers.get(weight.qweight)
    if hit is None or hit[0] != identity or hit[2] != weight.qweight._version:
        try:
            layer = pack_svdq_w4a4_linear(None, low_rank_down, low_rank_up, bias, packed_residual=weight.qweight,
                                          residual_scale=scales, dtype=activation.dtype, rotation=rotation,
                                          device=activation.device)
        except (TypeError, ValueError) as exc:
            raise XQTBackendError(f"B200 SVD W4A4 packing rejected: {exc}") from exc
        hit = (identity, layer, weight.qweight._version, (scales, low_rank_down, low_rank_up, bias))   # keeps the ids alive
        _svd_layers[weight.qweight] = hit
    result = svdq_w4a4_linear(activation.contiguous(), hit[1])
    if output is not None:
        output.copy_(result)
        return output
    return result


_EXECUTORS = {B200_W4A16: b200_w4a16_executor, B200_W8A8: b200_w8a8_executor, B200_SVD_W4A4: b200_svd_w4a4_executor}


def _rows_for(registry) -> tuple:
    """The B200 rows as instances of the row class the target registry already holds (xqt's own
    ``GemmKernelRegistration`` / ``GemmCapability`` when installing into xqt's table), else ours."""

    rows = b200_rows()
    try:
        sample = next(iter(registry.entries()))
    except (StopIteration, AttributeError, TypeError):
        return rows
    row_cls, cap_cls = type(sample), type(sample.capability)
    if row_cls is type(rows[0]):
        return rows
    row_fields, cap_fields = set(_field_names(row_cls)), set(_field_names(cap_cls))
    converted = []
    for row in rows:
        cap = cap_cls(**{f: getattr(row.capability, f) for f in _field_names(type(row.capability)) if f in cap_fields})
        values = {f: getattr(row, f) for f in _field_names(type(row)) if f in row_fields and f != "capability"}
        converted.append(row_cls(capability=cap, **values))
    return tuple(converted)


def _field_names(cls) -> tuple[str, ...]:
    return tuple(f.name for f in _dc_fields(cls))


def install_b200_executors(registry: GemmKernelRegistry | None = None, *, require_native: bool = True) -> tuple[str, ...]:
    """Register the B200 rows (if absent) and promote those with an executor to ``executable``.

    Returns the names promoted.  With ``require_native`` (default) a missing or stale shared
    library raises ``NativeLibraryError`` instead of silently leaving rows metadata-only.
    """

    from .registry import default_registry

    registry = default_registry() if registry is None else registry
    if require_native:
        native.library()
    elif not native.available():
        return ()
    promoted = []
    for row in _rows_for(registry):
        try:
            registry.get(row.name)
        except KeyError:
            registry.register(row)
        executor = _EXECUTORS.get(row.name)
        if executor is None:
            continue
        registry.replace(_dc_replace(registry.get(row.name), maturity="executable", executor=executor))
        promoted.append(row.name)
    return tuple(promoted)


__all__ = ["SVDGemmContract", "b200_svd_w4a4_executor", "b200_w4a16_executor", "b200_w8a8_executor", "install_b200_executors"]
