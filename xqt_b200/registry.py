"""GEMM kernel registry: the table the B200 executors are installed into.

Mirror of xqt's ``GemmCapability / GemmKernelRegistration / GemmKernelRegistry``
(xqt/kernels/ops/gemm/registry.py:17-213): same fields, same ``supports`` predicate, same
``register`` (conflict -> ValueError) / ``replace`` (unknown -> KeyError) / ``matching``
(priority-descending) behaviour, so the reference's registry tests read the same here.  The
rows themselves are new: xqt has no executable sm_100 row (its ladder stops at sm_89/sm_90/sm_120,
registry.py:845-977,1200-1383).  ``default_registry()`` holds the B200 rows as ``metadata_only``;
:func:`xqt_b200.executors.install_b200_executors` promotes them to ``executable`` the way
``install_sm89_w4a16_dequant_executor`` does (w4a16_sm89.py:303-340).  There are deliberately no
``reference_guarded`` CPU rows in this registry: this package ships no CPU fallback.
"""

from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any, Callable, Iterable

from .contracts import EpilogueSpec, GemmProblem, QuantSpec

MATURITIES = frozenset({"executable", "metadata_only", "planned", "reference_guarded", "experimental"})
SCOPES = frozenset({"contract", "precision"})
GemmExecutor = Callable[..., Any]


def _admits(allowed: tuple[str, ...], value: str, *, wildcard: bool = True) -> bool:
    """``value`` is listed, or the list holds the wildcard ``"any"`` (where one is honoured)."""

    return value in allowed or (wildcard and "any" in allowed)


@dataclass(frozen=True, slots=True)
class GemmCapability:
    """What a row can serve.  Field names and defaults are the schema xqt's dispatcher and reports read."""

    architectures: tuple[str, ...] = ("any",)
    weight_dtypes: tuple[str, ...] = ("fp32",)
    activation_dtypes: tuple[str, ...] = ("fp32",)
    scale_modes: tuple[str, ...] = ("w:none/a:none",)
    phases: tuple[str, ...] = ("generic", "prefill", "decode")
    epilogues: tuple[str, ...] = ("none",)
    min_sm: int | None = None

    def supports(self, problem: GemmProblem, quant: QuantSpec, epilogue: EpilogueSpec) -> bool:
        # dtypes are exact matches; architecture, scale mode, phase and epilogue accept "any"
        listed = (
            _admits(self.architectures, problem.arch),
            _admits(self.weight_dtypes, quant.weight_dtype, wildcard=False),
            _admits(self.activation_dtypes, quant.activation_dtype, wildcard=False),
            _admits(self.scale_modes, quant.scale_mode),
            _admits(self.phases, problem.phase),
            _admits(self.epilogues, epilogue.activation),
        )
        if not all(listed):
            return False
        return self.min_sm is None or (problem.sm is not None and problem.sm >= self.min_sm)

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {}
        for item in fields(self):
            value = getattr(self, item.name)
            out[item.name] = list(value) if isinstance(value, tuple) else value
        return out


@dataclass(frozen=True, slots=True)
class GemmKernelRegistration:
    """One row of the table: identity, capability, tuning metadata and (when executable) the callable."""

    name: str
    backend: str
    maturity: str
    capability: GemmCapability
    kernel_family: str
    layout: str = "canonical"
    tile_shape: tuple[int, int, int] | None = None
    warp_count: int | None = None
    stage_count: int | None = None
    alignment: tuple[int, int, int] = (1, 1, 1)
    priority: int = 0
    implementation: str = "reference"
    scope: str = "contract"
    selection_reason: str = ""
    executor: GemmExecutor | None = field(default=None, compare=False, repr=False)

    def __post_init__(self) -> None:
        problems = []
        if not self.name.strip():
            problems.append("name is empty")
        if self.maturity not in MATURITIES:
            problems.append(f"maturity {self.maturity!r} is not one of {sorted(MATURITIES)}")
        if self.scope not in SCOPES:
            problems.append(f"scope {self.scope!r} is not one of {sorted(SCOPES)}")
        if self.priority < 0:
            problems.append("priority is negative")
        for label, values in (("alignment", self.alignment), ("tile_shape", self.tile_shape or ())):
            if any(int(v) <= 0 for v in values):
                problems.append(f"{label} holds a non-positive entry")
        if self.maturity == "executable" and self.executor is None:
            problems.append("an executable row needs an executor")
        if problems:
            raise ValueError(f"GEMM registration {self.name!r}: " + "; ".join(problems))

    @property
    def executable(self) -> bool:
        return self.executor is not None and self.maturity == "executable"

    def supports(self, problem: GemmProblem, quant: QuantSpec, epilogue: EpilogueSpec) -> bool:
        return self.capability.supports(problem, quant, epilogue)

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {}
        for item in fields(self):
            if item.name in ("executor", "capability", "selection_reason"):
                continue
            value = getattr(self, item.name)
            out[item.name] = list(value) if isinstance(value, tuple) else value
        out["executable"] = self.executable
        out["capability"] = self.capability.to_dict()
        return out


class GemmKernelRegistry:
    """Rows by name, in insertion order.  ``register`` refuses a second, different row of the same
    name (ValueError; the identical row is a no-op), ``replace`` swaps an existing row (KeyError if
    there is none), ``matching`` lists the contract-scope rows that support a request, best priority first."""

    def __init__(self, entries: Iterable[GemmKernelRegistration] = ()) -> None:
        self._rows: dict[str, GemmKernelRegistration] = {}
        for row in entries:
            self.register(row)

    def register(self, entry: GemmKernelRegistration) -> None:
        present = self._rows.setdefault(entry.name, entry)
        if present is not entry and present != entry:
            raise ValueError(
                f"GEMM kernel {entry.name!r} is already registered with a different definition "
                f"(backend {present.backend!r}; the incoming row has backend {entry.backend!r})")

    def replace(self, entry: GemmKernelRegistration) -> None:
        self.get(entry.name)                     # KeyError when the row does not exist
        self._rows[entry.name] = entry

    def get(self, name: str) -> GemmKernelRegistration:
        row = self._rows.get(name)
        if row is None:
            raise KeyError(f"no GEMM kernel registration named {name!r}")
        return row

    def entries(self) -> tuple[GemmKernelRegistration, ...]:
        return tuple(self._rows.values())

    def matching(self, problem, quant, epilogue) -> tuple[GemmKernelRegistration, ...]:
        rows = (row for row in self._rows.values() if row.scope == "contract")
        able = [row for row in rows if row.supports(problem, quant, epilogue)]
        able.sort(key=lambda row: -row.priority)          # stable: insertion order breaks ties
        return tuple(able)

    def to_dict(self) -> list[dict[str, Any]]:
        return [row.to_dict() for row in self._rows.values()]


# ------------------------------------------------------------------------------- B200 rows

B200_W4A16 = "sm100_w4a16_b200"
B200_W8A8 = "sm100_w8a8_int8_b200"
B200_SVD_W4A4 = "sm100_svd_w4a4_b200"

_W4A16_SCALE_MODES = ("w:groupwise/a:per_tensor", "w:groupwise/a:none", "w:groupwise/a:per_token")


def b200_rows() -> tuple[GemmKernelRegistration, ...]:
    """The rows this backend adds.  Priorities sit above xqt's reference rows (5-8) and its
    sm_89 ladder does not match ``arch == 'sm_100'`` at all."""

    return (
        GemmKernelRegistration(
            name=B200_W4A16, backend="custom_cuda", maturity="metadata_only",
            capability=GemmCapability(
                architectures=("sm_100",), weight_dtypes=("int4",), activation_dtypes=("fp16", "bf16"),
                scale_modes=_W4A16_SCALE_MODES, epilogues=("none", "relu", "gelu", "silu"), min_sm=100),
            kernel_family="w4a16_b200", layout="xqt_int4_nk_v1", tile_shape=(128, 128, 64), warp_count=8,
            stage_count=4, priority=60, implementation="cuda_sm100a_w4a16",
            selection_reason="M<=16: split-K tensor-core GEMV; larger M: TMA + tcgen05 dequant GEMM",
        ),
        GemmKernelRegistration(
            name=B200_W8A8, backend="custom_cuda", maturity="metadata_only",
            capability=GemmCapability(
                architectures=("sm_100",), weight_dtypes=("int8",), activation_dtypes=("int8",),
                scale_modes=("w:per_channel/a:per_token", "w:per_channel/a:per_tensor"), epilogues=("none",), min_sm=100),
            kernel_family="w8a8_int8_b200", layout="xqt_int8_nk_v1", tile_shape=(128, 256, 128), warp_count=6,
            stage_count=4, priority=60, implementation="cuda_sm100a_w8a8",
            selection_reason="per-token int8 quantisation prologue + tcgen05 kind::i8 GEMM, fp32 dequant epilogue",
        ),
        GemmKernelRegistration(
            name=B200_SVD_W4A4, backend="custom_cuda", maturity="metadata_only",
            capability=GemmCapability(
                architectures=("sm_100",), weight_dtypes=("int4",), activation_dtypes=("fp16", "bf16"),
                scale_modes=("w:groupwise/a:per_token", "w:groupwise/a:per_tensor", "w:groupwise/a:none"),
                epilogues=("none",), min_sm=100),
            kernel_family="svd_w4a4_b200", layout="xqt_int4_nk_v1", tile_shape=(128, 128, 64), warp_count=8,
            stage_count=4, priority=55, implementation="cuda_sm100a_svd_w4a4",
            selection_reason="int4 residual + rank-r pair (executor kwargs low_rank_down / low_rank_up): group-64 int4 "
                             "activations quantised in the call, kind::i8 GEMM, low-rank up projection in the epilogue; "
                             "below the W4A16 row, which serves the same request without a low-rank pair",
        ),
    )


_default: GemmKernelRegistry | None = None


def default_registry() -> GemmKernelRegistry:
    global _default
    if _default is None:
        _default = GemmKernelRegistry(b200_rows())
    return _default


__all__ = [
    "B200_SVD_W4A4", "B200_W4A16", "B200_W8A8", "GemmCapability", "GemmExecutor", "GemmKernelRegistration",
    "GemmKernelRegistry", "b200_rows", "default_registry",
]
