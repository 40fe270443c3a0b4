"""Registry-driven GEMM dispatch with an explicit selection report.

Mirror of xqt's ``dispatch_gemm`` (xqt/kernels/ops/gemm/dispatch.py:155-360): candidates are the
registry rows that support the problem, in priority order, with a requested kernel moved to the
front; rows that are not executable are skipped with a recorded reason; an executor that raises
``XQTBackendError`` is recorded and the next candidate is tried.  xqt ends that ladder in its torch
reference; this package has no CPU path, so when nothing executable is left the call raises the
same ``RuntimeError`` xqt raises for ``allow_reference=False`` (dispatch.py:262-270).
"""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any, Mapping

import torch

from .contracts import GemmSpec, PackedWeight
from .errors import XQTBackendError
from .layout import W4_LAYOUT, validate_w4a16_packed_weight
from .registry import GemmKernelRegistry, default_registry


@dataclass(frozen=True, slots=True)
class GemmDispatchReport:
    requested_kernel: str | None
    selected_kernel: str
    backend: str
    kernel_family: str
    maturity: str
    arch: str
    tile_shape: tuple[int, int, int] | None
    warp_count: int | None
    stage_count: int | None
    scale_mode: str
    pack_version: str
    weight_scale_source: str = "none"
    activation_scale_source: str = "none"
    activation_granularity: str = "none"
    padding_ratio: float = 0.0
    fallback_reason: str | None = None
    fallback_chain: tuple[str, ...] = ()
    group_size: int | None = None
    native: bool = False
    shape_variant: str = "generic"

    def to_dict(self) -> dict[str, Any]:
        payload = asdict(self)
        payload["tile_shape"] = None if self.tile_shape is None else list(self.tile_shape)
        payload["fallback_chain"] = list(self.fallback_chain)
        return payload


@dataclass(frozen=True, slots=True)
class GemmDispatchResult:
    output: torch.Tensor
    report: GemmDispatchReport


def dispatch_gemm(
    activation: torch.Tensor,
    weight: torch.Tensor | PackedWeight,
    *,
    spec: GemmSpec,
    weight_scales: torch.Tensor | None = None,
    activation_scales: torch.Tensor | None = None,
    weight_zero_points: torch.Tensor | None = None,
    activation_zero_points: torch.Tensor | None = None,
    bias: torch.Tensor | None = None,
    residual: torch.Tensor | None = None,
    registry: GemmKernelRegistry | None = None,
    requested_kernel: str | None = None,
    candidate_kernels: tuple[str, ...] | None = None,
    executor_kwargs: Mapping[str, Any] | None = None,
    allow_reference: bool = False,
) -> GemmDispatchResult:
    if not isinstance(spec, GemmSpec):
        raise TypeError("dispatch_gemm requires a complete GemmSpec")
    if allow_reference:
        raise XQTBackendError("the B200 backend ships no CPU reference path; allow_reference must stay False")
    active = default_registry() if registry is None else registry
    all_matches = active.matching(spec.problem, spec.quant, spec.epilogue)
    if candidate_kernels is not None:
        matches = tuple(active.get(name) for name in candidate_kernels)
        bad = tuple(e.name for e in matches if not e.supports(spec.problem, spec.quant, spec.epilogue))
        if bad:
            raise ValueError(f"candidate kernels do not support problem/quant/epilogue: {bad}")
    elif requested_kernel is not None:
        requested = active.get(requested_kernel)
        if not requested.supports(spec.problem, spec.quant, spec.epilogue):
            raise ValueError(f"requested kernel {requested_kernel!r} does not support problem/quant/epilogue")
        matches = (requested,) + tuple(e for e in all_matches if e.name != requested.name)
    else:
        matches = all_matches
    if not matches:
        raise RuntimeError(
            "no GEMM registry entry supports "
            f"arch={spec.problem.arch}, weight_dtype={spec.quant.weight_dtype}, "
            f"activation_dtype={spec.quant.activation_dtype}, scale_mode={spec.quant.scale_mode}"
        )
    packed = hasattr(weight, "metadata")
    if (
        spec.quant.weight_dtype == "int4" and packed and weight.metadata.storage_layout == W4_LAYOUT
        and spec.quant.activation_dtype in {"fp16", "bf16"}
    ):
        validate_w4a16_packed_weight(weight, spec=spec.quant, logical_shape=(spec.problem.n, spec.problem.k))
    reasons: list[str] = []
    chosen, output = None, None
    for candidate in matches:
        if not candidate.executable:
            if candidate.maturity in {"metadata_only", "planned"}:
                reasons.append(f"candidate {candidate.name!r} is maturity={candidate.maturity}")
            continue
        try:
            output = candidate.executor(
                activation, weight, spec=spec, weight_scales=weight_scales, activation_scales=activation_scales,
                weight_zero_points=weight_zero_points, activation_zero_points=activation_zero_points,
                bias=bias, residual=residual, **dict(executor_kwargs or {}),
            )
            chosen = candidate
        except XQTBackendError as exc:
            reasons.append(f"candidate {candidate.name!r} unavailable: {exc}")
            continue
        break
    if chosen is None or output is None:
        top = matches[0]
        details = "; ".join(reasons)
        raise RuntimeError(
            f"GEMM kernel {top.name!r} is maturity={top.maturity}, and no executable/reference fallback "
            f"is allowed" + (f" ({details})" if details else "")
        )
    align = chosen.alignment
    padded = [-(-dim // a) * a for dim, a in zip(spec.problem.shape, align)]
    logical = max(1, spec.problem.m * spec.problem.n * spec.problem.k)
    variant = "generic"
    if chosen.kernel_family == "w4a16_b200":
        variant = "gemv_m_le_16" if spec.problem.m <= 16 else "tcgen05_dequant_gemm"
    report = GemmDispatchReport(
        requested_kernel=requested_kernel, selected_kernel=chosen.name, backend=chosen.backend,
        kernel_family=chosen.kernel_family, maturity=chosen.maturity, arch=spec.problem.arch,
        tile_shape=chosen.tile_shape, warp_count=chosen.warp_count, stage_count=chosen.stage_count,
        scale_mode=spec.quant.scale_mode,
        pack_version=weight.metadata.pack_version if packed else spec.quant.pack_version,
        weight_scale_source=spec.quant.weight_scale_source,
        activation_scale_source=spec.quant.activation_scale_source,
        activation_granularity=spec.quant.activation_granularity,
        padding_ratio=float(padded[0] * padded[1] * padded[2] - logical) / float(logical),
        fallback_reason="; ".join(reasons) if reasons else None,
        fallback_chain=tuple(e.name for e in matches),
        group_size=weight.metadata.group_size if packed else spec.quant.group_size,
        native=True, shape_variant=variant,
    )
    return GemmDispatchResult(output=output, report=report)


def select_kernel(spec: GemmSpec, *, registry: GemmKernelRegistry | None = None):
    active = default_registry() if registry is None else registry
    return active.matching(spec.problem, spec.quant, spec.epilogue)


__all__ = ["GemmDispatchReport", "GemmDispatchResult", "dispatch_gemm", "select_kernel"]
