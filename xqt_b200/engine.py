"""Operator-stage integration: the ``b200_cuda`` engine, its materializer and the acceptance gate.

In xqt a YAML ``kind: operator`` stage names an engine per target; the engine's registration
(``EngineRegistration``, xqt/kernels/engine_resolve.py:48-82) says what it provides and which
materializer builds the candidate model (xqt/kernels/wrappers/materialize.py:52-92); the stage then
validates the candidate against the eager module (``validate{atol,rtol}``) and keeps it only if it is
faster than ``min_speedup`` (xqt/kernels/wrappers/types.py:11-35, execute.py:112-429).

This module supplies those three pieces for B200:

* :data:`B200_ENGINE` / :func:`register_b200_engine` -- the registration, handed to xqt's own
  ``register_engine`` when xqt is importable (same field names), kept locally otherwise;
* :func:`build_b200_candidate_model` / :func:`materialize_operator_candidate_model` -- the
  materializer: every sub-module of the target that exposes the packed-int4 bridge
  ``triton_packed_dequant_gemm_args`` is replaced by :class:`xqt_b200.modules.B200PackedDequantLinear`
  (pattern ``gemm_int4_dequant``); xqt's ``materialize.py`` dispatches on the registration's
  ``materializer`` name, so a one-line branch ``if materializer == "b200_cuda": return
  build_b200_candidate_model(target_model, target), None`` there wires it in;
* :func:`accept_candidate` -- numeric validation against the eager module and the speed-up gate, with
  the report fields the stage writes.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Optional

import torch
from torch import nn

from .errors import XQTBackendError
from .modules import B200PackedDequantLinear

# the patterns xqt's operator contract allows for the "linear" family that this engine serves
# (xqt/kernels/engine_resolve.py:344-361)
SERVED_LINEAR_PATTERNS = frozenset({"linear", "dequant_gemm_epilogue", "gemm_int4_dequant"})


@dataclass(frozen=True)
class EngineRegistration:
    """Field-for-field the schema of xqt's ``EngineRegistration`` (engine_resolve.py:48-82)."""

    name: str
    provides: frozenset
    min_capability: Optional[int] = None
    priority: int = 100
    dispatchable: bool = True
    maturity: str = "executable"
    status: str = "available"
    runtime: str = "pytorch"
    artifact_kind: str = "pytorch_model"
    exportable: bool = False
    requires_cuda: bool = False
    requires_calibration: bool = False
    requires_exportable_graph: bool = False
    operator_visible: bool = False
    operator_order: int = 999
    convert_visible: bool = False
    convert_order: int = 999
    materializer: Optional[str] = None
    recommended_patterns: frozenset = frozenset()
    required_packages: tuple = ()
    notes: tuple = ()
    limitations: tuple = ()


B200_ENGINE = EngineRegistration(
    name="b200_cuda",
    provides=frozenset({"int8_mma", "true_int8_mma", "int4_mma", "dequant_gemm_epilogue", "hadamard_groupwise",
                        "w4_storage_int8_mma", "gemm_int4_dequant"}),
    min_capability=100, priority=60, requires_cuda=True, operator_visible=True, operator_order=20,
    materializer="b200_cuda", recommended_patterns=frozenset({"dequant_gemm_epilogue", "gemm_int4_dequant"}),
    required_packages=("torch",),
    notes=("Hand-written sm_100a kernels behind a C ABI (libxqt_b200.so); no just-in-time compilation.",),
    limitations=("Serves packed int4 weight-only linears (group 32/64/128); other module kinds keep their eager form.",),
)

_local_engines: dict[str, EngineRegistration] = {}


def register_b200_engine() -> Any:
    """Register the engine with xqt's engine table when xqt is importable (returns xqt's registration
    object), else in this package's own table (returns :data:`B200_ENGINE`)."""

    try:
        from xqt.kernels import engine_resolve as xer
    except Exception:  # noqa: BLE001 - xqt absent (or its optional imports are): keep the local table
        _local_engines[B200_ENGINE.name] = B200_ENGINE
        return B200_ENGINE
    theirs = {f: getattr(B200_ENGINE, f) for f in B200_ENGINE.__dataclass_fields__
              if f in xer.EngineRegistration.__dataclass_fields__}
    return xer.register_engine(xer.EngineRegistration(**theirs))


def get_engine_registration(name: str) -> EngineRegistration | None:
    return _local_engines.get(name) or (B200_ENGINE if name == B200_ENGINE.name else None)


@dataclass
class OperatorOptimizationTargetPlan:
    """The fields of xqt's target plan this engine reads (xqt/kernels/wrappers/types.py:11-35)."""

    name: str
    engine: str = "b200_cuda"
    target_path: Optional[str] = None
    candidate_kind: str = "single_kernel"
    options: dict = field(default_factory=dict)
    patterns: list = field(default_factory=list)
    fallback: str = "eager"
    fallback_policy: str = "prefer_fallback"
    min_speedup: float = 1.01
    validate: dict = field(default_factory=dict)


def _is_packed_int4_linear(module: nn.Module) -> bool:
    return callable(getattr(module, "triton_packed_dequant_gemm_args", None))


def build_b200_candidate_model(target_model: nn.Module, target: Any) -> nn.Module:
    """The materializer: replace every packed-int4 linear inside ``target_model`` (or the model itself)."""

    patterns = set(getattr(target, "patterns", None) or ())
    unsupported = patterns - SERVED_LINEAR_PATTERNS
    if unsupported:
        raise XQTBackendError(f"Operator optimization engine 'b200_cuda' does not serve patterns {sorted(unsupported)}")
    fallback = str(getattr(target, "fallback", "eager"))
    settings = dict(getattr(target, "options", None) or {})
    if _is_packed_int4_linear(target_model):
        return B200PackedDequantLinear(target_model, fallback=fallback, settings=settings)
    replaced = 0
    for parent in list(target_model.modules()):
        for child_name, child in list(parent.named_children()):
            if _is_packed_int4_linear(child) and not isinstance(child, B200PackedDequantLinear):
                setattr(parent, child_name, B200PackedDequantLinear(child, fallback=fallback, settings=settings))
                replaced += 1
    if replaced == 0:
        raise XQTBackendError("Operator optimization engine 'b200_cuda' found no packed int4 linear in the target")
    return target_model


def materialize_operator_candidate_model(model: nn.Module, target: Any) -> tuple[nn.Module, float | None]:
    """One candidate root model with the target's replacement applied (materialize.py:80-92): the root is
    deep-copied, the sub-module at ``target.target_path`` is rebuilt, compile time is ``None``."""

    root = copy.deepcopy(model)
    path = getattr(target, "target_path", None)
    if not path:
        return build_b200_candidate_model(root, target), None
    parent_path, _, attribute = path.rpartition(".")
    parent = root.get_submodule(parent_path) if parent_path else root
    replacement = build_b200_candidate_model(root.get_submodule(path), target)
    if attribute.isdigit() and isinstance(parent, (nn.Sequential, nn.ModuleList)):
        parent[int(attribute)] = replacement
    else:
        setattr(parent, attribute, replacement)
    return root, None


def _time_ms(fn, reps: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / reps


def accept_candidate(eager: nn.Module, candidate: nn.Module, sample: torch.Tensor, target: Any, *, reps: int = 20) -> dict:
    """The stage's acceptance gate: ``validate{atol, rtol}`` against the eager module on ``sample``, then the
    measured speed-up against ``min_speedup``; ``fallback_policy == "prefer_fallback"`` keeps the eager
    module unless both hold."""

    validate = dict(getattr(target, "validate", None) or {})
    atol, rtol = float(validate.get("atol", 1e-2)), float(validate.get("rtol", 1e-2))
    with torch.no_grad():
        want, got = eager(sample), candidate(sample)
    error = (got.float() - want.float()).abs()
    bound = atol + rtol * want.float().abs()
    numerics_ok = bool((error <= bound).all())
    speedup = None
    if sample.is_cuda and numerics_ok:
        with torch.no_grad():
            speedup = _time_ms(lambda: eager(sample), reps) / max(_time_ms(lambda: candidate(sample), reps), 1e-9)
    fast_enough = speedup is not None and speedup >= float(getattr(target, "min_speedup", 1.01))
    accepted = numerics_ok and (fast_enough or getattr(target, "fallback_policy", "prefer_fallback") != "prefer_fallback")
    return {
        "target": getattr(target, "name", None), "engine": B200_ENGINE.name, "accepted": bool(accepted),
        "numerics_ok": numerics_ok, "max_abs_error": float(error.max()), "atol": atol, "rtol": rtol,
        "speedup": speedup, "min_speedup": float(getattr(target, "min_speedup", 1.01)),
        "fallback": getattr(target, "fallback", "eager"),
        "execution_metadata": [m.execution_metadata() for m in candidate.modules() if isinstance(m, B200PackedDequantLinear)],
    }


__all__ = ["B200_ENGINE", "EngineRegistration", "OperatorOptimizationTargetPlan", "SERVED_LINEAR_PATTERNS", "accept_candidate",
           "build_b200_candidate_model", "get_engine_registration", "materialize_operator_candidate_model",
           "register_b200_engine"]
