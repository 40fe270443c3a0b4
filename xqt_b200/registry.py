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

from dataclasses import dataclass, field
from typing import Any, Callable, Iterable

from .contracts import EpilogueSpec, GemmProblem, QuantSpec

MATURITIES = frozenset({"executable", "metadata_only", "planned", "reference_guarded", "experimental"})
GemmExecutor = Callable[..., Any]


@dataclass(frozen=True, slots=True)
class GemmCapability:
    architectures: tuple[str, ...] = ("any",)
    weight_dtypes: tuple[str, ...] = ("fp32",)
    activation_dtypes: tuple[str, ...] = ("fp32",)
    scale_modes: tuple[str, ...] = ("w:none/a:none",)
    phases: tuple[str, ...] = ("generic", "prefill", "decode")
    epilogues: tuple[str, ...] = ("none",)
    min_sm: int | None = None

    def supports(self, problem: GemmProblem, quant: QuantSpec, epilogue: EpilogueSpec) -> bool:
        if "any" not in self.architectures and problem.arch not in self.architectures:
            return False
        if quant.weight_dtype not in self.weight_dtypes:
            return False
        if quant.activation_dtype not in self.activation_dtypes:
            return False
        if quant.scale_mode not in self.scale_modes and "any" not in self.scale_modes:
            return False
        if problem.phase not in self.phases and "any" not in self.phases:
            return False
        if epilogue.activation not in self.epilogues and "any" not in self.epilogues:
            return False
        if self.min_sm is not None and (problem.sm is None or problem.sm < self.min_sm):
            return False
        return True

    def to_dict(self) -> dict[str, Any]:
        return {
            "architectures": list(self.architectures),
            "weight_dtypes": list(self.weight_dtypes),
            "activation_dtypes": list(self.activation_dtypes),
            "scale_modes": list(self.scale_modes),
            "phases": list(self.phases),
            "epilogues": list(self.epilogues),
            "min_sm": self.min_sm,
        }


@dataclass(frozen=True, slots=True)
class GemmKernelRegistration:
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
        if not self.name.strip():
            raise ValueError("GemmKernelRegistration.name must be non-empty")
        if self.maturity not in MATURITIES:
            raise ValueError(f"unsupported GEMM maturity: {self.maturity!r}")
        if self.priority < 0:
            raise ValueError("kernel priority must be non-negative")
        if any(int(item) <= 0 for item in self.alignment):
            raise ValueError("kernel alignment values must be positive")
        if self.tile_shape is not None and any(int(item) <= 0 for item in self.tile_shape):
            raise ValueError("tile_shape values must be positive")
        if self.maturity == "executable" and self.executor is None:
            raise ValueError("executable GEMM registration requires an executor")
        if self.scope not in {"contract", "precision"}:
            raise ValueError("GEMM registration scope must be contract or precision")

    @property
    def executable(self) -> bool:
        return self.maturity == "executable" and self.executor is not None

    def supports(self, problem: GemmProblem, quant: QuantSpec, epilogue: EpilogueSpec) -> bool:
        return self.capability.supports(problem, quant, epilogue)

    def to_dict(self) -> dict[str, Any]:
        return {
            "name": self.name,
            "backend": self.backend,
            "maturity": self.maturity,
            "kernel_family": self.kernel_family,
            "layout": self.layout,
            "tile_shape": None if self.tile_shape is None else list(self.tile_shape),
            "warp_count": self.warp_count,
            "stage_count": self.stage_count,
            "alignment": list(self.alignment),
            "priority": self.priority,
            "implementation": self.implementation,
            "scope": self.scope,
            "executable": self.executable,
            "capability": self.capability.to_dict(),
        }


class GemmKernelRegistry:
    def __init__(self, entries: Iterable[GemmKernelRegistration] = ()) -> None:
        self._entries: dict[str, GemmKernelRegistration] = {}
        for entry in entries:
            self.register(entry)

    def register(self, entry: GemmKernelRegistration) -> None:
        existing = self._entries.get(entry.name)
        if existing is not None:
            if existing == entry:
                return
            raise ValueError(
                f"Conflicting GEMM kernel registration for {entry.name!r}: "
                f"existing backend={existing.backend!r}, incoming backend={entry.backend!r}"
            )
        self._entries[entry.name] = entry

    def replace(self, entry: GemmKernelRegistration) -> None:
        if entry.name not in self._entries:
            raise KeyError(f"cannot replace unknown GEMM kernel registration: {entry.name!r}")
        self._entries[entry.name] = entry

    def get(self, name: str) -> GemmKernelRegistration:
        try:
            return self._entries[name]
        except KeyError as exc:
            raise KeyError(f"unknown GEMM kernel registration: {name!r}") from exc

    def entries(self) -> tuple[GemmKernelRegistration, ...]:
        return tuple(self._entries.values())

    def matching(self, problem, quant, epilogue) -> tuple[GemmKernelRegistration, ...]:
        found = [e for e in self._entries.values() if e.scope == "contract" and e.supports(problem, quant, epilogue)]
        return tuple(sorted(found, key=lambda e: e.priority, reverse=True))

    def to_dict(self) -> list[dict[str, Any]]:
        return [entry.to_dict() for entry in self.entries()]


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
                scale_modes=("w:per_channel/a:per_token",), epilogues=("none",), min_sm=100),
            kernel_family="w8a8_int8_b200", layout="xqt_int8_nk_v1", tile_shape=(128, 256, 128), warp_count=6,
            stage_count=4, priority=60, implementation="cuda_sm100a_w8a8",
            selection_reason="per-token int8 quantisation prologue + tcgen05 kind::i8 GEMM, fp32 dequant epilogue",
        ),
        GemmKernelRegistration(
            name=B200_SVD_W4A4, backend="custom_cuda", maturity="metadata_only",
            capability=GemmCapability(
                architectures=("sm_100",), weight_dtypes=("int4",), activation_dtypes=("int8",),
                scale_modes=("w:groupwise/a:per_token",), epilogues=("none",), min_sm=100),
            kernel_family="svd_w4a4_b200", layout="xqt_int4_nk_v1", tile_shape=(128, 128, 64), warp_count=8,
            stage_count=4, priority=60, implementation="cuda_sm100a_svd_w4a4",
            selection_reason="rotation + group-64 int4 activations, kind::i8 GEMM, rank-r low-rank branch",
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
