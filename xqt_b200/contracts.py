"""Logical GEMM contracts of the quantized-linear path.

Host-side mirror of xqt's GEMM contract types (xqt/kernels/ops/gemm/contracts.py:75-491):
same class names, field names, defaults and validation outcomes, so that code and
tests written against xqt's ``GemmProblem / QuantSpec / EpilogueSpec / GemmSpec /
PackedWeight`` read the same against this package.  The convention is always
``Y[M,N] = A[M,K] @ W[N,K].T``.  Duck typing is deliberate: the executors in
:mod:`xqt_b200.executors` only read attributes, so xqt's own dataclasses can be
passed in as well.
"""

from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any, Mapping, Sequence

import torch

DTYPE_NAMES = frozenset(
    "fp32 int32 fp16 bf16 int8 int4 int3 int2 fp8_e4m3 fp8_e5m2 fp4 mxfp8 mxfp6 mxfp4 nvfp4 codebook none".split()
)
GRANULARITIES = frozenset({"none", "per_tensor", "per_channel", "per_token", "groupwise", "blockwise"})
SCALE_SOURCES = frozenset(
    {"none", "weight_offline", "weight_load_time", "activation_static", "activation_dynamic"}
)
_QUANTIZED_WEIGHT_DTYPES = DTYPE_NAMES - {"fp32", "int32", "fp16", "bf16", "none"}
_QUANTIZED_ACT_DTYPES = frozenset({"int8", "fp8_e4m3", "fp8_e5m2"})
_FP8 = frozenset({"fp8_e4m3", "fp8_e5m2"})


def _positive_int(owner: str, name: str, value: Any, *, allow_zero: bool = False) -> int:
    if isinstance(value, bool) or int(value) != value:
        raise ValueError(f"{owner}.{name} must be an int")
    number = int(value)
    if number < 0 or (number == 0 and not allow_zero):
        bound = "non-negative" if allow_zero else "positive"
        raise ValueError(f"{owner}.{name} must be a {bound} int")
    return number


def _shape2(value: Sequence[int], name: str) -> tuple[int, int]:
    if not isinstance(value, (list, tuple)):
        raise TypeError(f"{name} must be a sequence of ints")
    if len(value) != 2:
        raise ValueError(f"{name} must have rank 2, got {len(value)}")
    out = []
    for item in value:
        if isinstance(item, bool):
            raise TypeError(f"{name} entries must be positive ints")
        number = int(item)
        if number <= 0:
            raise ValueError(f"{name} entries must be positive, got {number}")
        out.append(number)
    return out[0], out[1]


@dataclass(frozen=True, slots=True)
class GemmProblem:
    """Logical problem; only M may be zero (contracts.py:75-137)."""

    m: int
    n: int
    k: int
    op: str = "dense"
    phase: str = "generic"
    batch: int = 1
    group_count: int = 1
    device: str = "cpu"
    sm: int | None = None
    cuda_graph: bool = False

    def __post_init__(self) -> None:
        set_ = object.__setattr__
        for name in ("n", "k", "batch", "group_count"):
            set_(self, name, _positive_int("GemmProblem", name, getattr(self, name)))
        set_(self, "m", _positive_int("GemmProblem", "m", self.m, allow_zero=True))
        if self.op not in {"dense", "batched", "grouped"}:
            raise ValueError(f"GemmProblem.op unsupported: {self.op!r}")
        if self.phase not in {"generic", "prefill", "decode"}:
            raise ValueError(f"GemmProblem.phase unsupported: {self.phase!r}")
        if not str(self.device):
            raise ValueError("GemmProblem.device must be a non-empty string")
        set_(self, "device", str(self.device))
        if self.sm is not None:
            set_(self, "sm", _positive_int("GemmProblem", "sm", self.sm, allow_zero=True))
        if not isinstance(self.cuda_graph, bool):
            raise TypeError("GemmProblem.cuda_graph must be bool")

    @property
    def shape(self) -> tuple[int, int, int]:
        return self.m, self.n, self.k

    @property
    def arch(self) -> str:
        return "unknown" if self.sm is None else f"sm_{self.sm}"

    def to_dict(self) -> dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in fields(self)}

    @classmethod
    def from_dict(cls, payload: Mapping[str, Any]) -> "GemmProblem":
        if not isinstance(payload, Mapping):
            raise TypeError("GemmProblem.from_dict expects a mapping")
        known = {f.name for f in fields(cls)}
        return cls(**{key: value for key, value in payload.items() if key in known})


@dataclass(frozen=True, slots=True)
class QuantSpec:
    """Quantization side of the contract (contracts.py:166-305)."""

    weight_dtype: str = "fp16"
    activation_dtype: str = "fp16"
    compute_dtype: str = "fp32"
    accum_dtype: str = "fp32"
    output_dtype: str = "fp16"
    weight_granularity: str = "per_tensor"
    activation_granularity: str = "per_tensor"
    group_axis: str = "k"
    group_size: int | None = None
    symmetric: bool = True
    weight_zero_point: bool = False
    activation_zero_point: bool = False
    weight_scale_source: str = "none"
    activation_scale_source: str = "none"
    storage_layout: str = "canonical"
    pack_version: str = "canonical-v1"

    def __post_init__(self) -> None:
        set_ = object.__setattr__
        for name in ("weight_dtype", "activation_dtype", "compute_dtype", "accum_dtype", "output_dtype"):
            value = str(getattr(self, name))
            if value not in DTYPE_NAMES:
                raise ValueError(f"QuantSpec.{name} unsupported dtype: {value!r}")
            set_(self, name, value)
        for name in ("weight_granularity", "activation_granularity"):
            value = str(getattr(self, name))
            if value not in GRANULARITIES:
                raise ValueError(f"QuantSpec.{name} unsupported value: {value!r}")
            set_(self, name, value)
        if self.group_axis not in {"k", "n", "m"}:
            raise ValueError("QuantSpec.group_axis must be 'k', 'n', or 'm'")
        if self.weight_granularity in {"groupwise", "blockwise"}:
            if self.group_size is None or int(self.group_size) <= 0:
                raise ValueError("groupwise/blockwise weight quantization requires group_size > 0")
            set_(self, "group_size", int(self.group_size))
        elif self.group_size is not None:
            raise ValueError("group_size is only valid for groupwise/blockwise weights")
        for name in ("symmetric", "weight_zero_point", "activation_zero_point"):
            if not isinstance(getattr(self, name), bool):
                raise TypeError(f"QuantSpec.{name} must be bool")
        if self.weight_dtype in _FP8 and (not self.symmetric or self.weight_zero_point):
            raise ValueError("FP8 weights are signed and carry no integer zero point")
        if self.activation_dtype in _FP8 and self.activation_zero_point:
            raise ValueError("FP8 activations do not support integer zero points")
        for name in ("weight_scale_source", "activation_scale_source"):
            value = str(getattr(self, name))
            if value not in SCALE_SOURCES:
                raise ValueError(f"QuantSpec.{name} unsupported value: {value!r}")
            set_(self, name, value)
        if self.weight_dtype in _QUANTIZED_WEIGHT_DTYPES:
            if self.weight_scale_source == "none":
                raise ValueError("quantized weights require weight_scale_source")
        elif self.weight_scale_source != "none":
            raise ValueError("dense weights cannot declare a weight scale source")
        if self.activation_dtype in _QUANTIZED_ACT_DTYPES:
            if self.activation_scale_source not in {"activation_static", "activation_dynamic"}:
                raise ValueError(
                    "QuantSpec.activation_scale_source must be activation_static "
                    "or activation_dynamic for quantized activations"
                )
        elif self.activation_scale_source != "none":
            raise ValueError("non-quantized activations cannot declare an activation scale source")
        for name in ("storage_layout", "pack_version"):
            value = str(getattr(self, name)).strip()
            if not value:
                raise ValueError(f"QuantSpec.{name} must be non-empty")
            set_(self, name, value)

    @property
    def scale_mode(self) -> str:
        return f"w:{self.weight_granularity}/a:{self.activation_granularity}"

    @property
    def is_weight_only(self) -> bool:
        return self.activation_dtype not in _QUANTIZED_ACT_DTYPES

    def to_dict(self) -> dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in fields(self)}

    @classmethod
    def from_dict(cls, payload: Mapping[str, Any]) -> "QuantSpec":
        if not isinstance(payload, Mapping):
            raise TypeError("QuantSpec.from_dict expects a mapping")
        known = {f.name for f in fields(cls)}
        return cls(**{key: value for key, value in payload.items() if key in known})


@dataclass(frozen=True, slots=True)
class EpilogueSpec:
    """Post-accumulation operations (contracts.py:308-343)."""

    activation: str = "none"
    has_bias: bool = False
    has_residual: bool = False
    output_dtype: str = "fp16"

    def __post_init__(self) -> None:
        if self.activation not in {"none", "relu", "gelu", "silu"}:
            raise ValueError("EpilogueSpec.activation must be one of none/relu/gelu/silu")
        if not isinstance(self.has_bias, bool) or not isinstance(self.has_residual, bool):
            raise TypeError("EpilogueSpec.has_bias and has_residual must be bool")
        if self.output_dtype not in {"fp32", "fp16", "bf16"}:
            raise ValueError("EpilogueSpec.output_dtype must be fp32, fp16, or bf16")

    def to_dict(self) -> dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in fields(self)}

    @classmethod
    def from_dict(cls, payload: Mapping[str, Any]) -> "EpilogueSpec":
        if not isinstance(payload, Mapping):
            raise TypeError("EpilogueSpec.from_dict expects a mapping")
        known = {f.name for f in fields(cls)}
        return cls(**{key: value for key, value in payload.items() if key in known})


@dataclass(frozen=True, slots=True)
class GemmSpec:
    """Problem + quantization + epilogue (contracts.py:346-376)."""

    problem: GemmProblem
    quant: QuantSpec = field(default_factory=QuantSpec)
    epilogue: EpilogueSpec = field(default_factory=EpilogueSpec)

    def __post_init__(self) -> None:
        if self.epilogue.output_dtype != self.quant.output_dtype:
            raise ValueError("GemmSpec epilogue.output_dtype must match quant.output_dtype")

    def to_dict(self) -> dict[str, Any]:
        return {
            "problem": self.problem.to_dict(),
            "quant": self.quant.to_dict(),
            "epilogue": self.epilogue.to_dict(),
        }

    @classmethod
    def from_dict(cls, payload: Mapping[str, Any]) -> "GemmSpec":
        if not isinstance(payload, Mapping):
            raise TypeError("GemmSpec.from_dict expects a mapping")
        return cls(
            problem=GemmProblem.from_dict(payload["problem"]),
            quant=QuantSpec.from_dict(payload.get("quant", {})),
            epilogue=EpilogueSpec.from_dict(payload.get("epilogue", {})),
        )


@dataclass(frozen=True, slots=True)
class PackedWeightMetadata:
    """What makes a packed weight reversible and dispatchable (contracts.py:366-448).

    ``local_shape`` / ``shard_axis`` record a column (axis 0, over N) or row
    (axis 1, over K) partition of the logical weight across GPUs; xqt declares
    the fields (contracts.py:379-380) and this package's tensor-parallel layer
    is what fills and consumes them.
    """

    logical_shape: tuple[int, int]
    storage_layout: str
    pack_version: str
    weight_dtype: str
    padded_k: int
    group_size: int | None = None
    packed_bits: int | None = None
    nibble_order: str | None = None
    nibble_signed: bool = True
    local_shape: tuple[int, int] | None = None
    shard_axis: int | None = None
    global_scale: torch.Tensor | None = None

    def __post_init__(self) -> None:
        set_ = object.__setattr__
        logical = _shape2(self.logical_shape, "PackedWeightMetadata.logical_shape")
        set_(self, "logical_shape", logical)
        if int(self.padded_k) < logical[1]:
            raise ValueError("padded_k cannot be smaller than logical K")
        set_(self, "padded_k", int(self.padded_k))
        if self.weight_dtype not in DTYPE_NAMES:
            raise ValueError(f"unsupported packed weight dtype: {self.weight_dtype!r}")
        if self.packed_bits not in {None, 2, 3, 4, 8}:
            raise ValueError("packed_bits must be None, 2, 3, 4, or 8")
        if self.packed_bits == 4 and self.nibble_order not in {"low_high", "high_low"}:
            raise ValueError("4-bit weights require nibble_order low_high or high_low")
        if self.packed_bits in {2, 3} and self.nibble_order is not None:
            raise ValueError("2/3-bit weights do not use nibble_order")
        if not isinstance(self.nibble_signed, bool):
            raise TypeError("nibble_signed must be bool")
        if self.local_shape is not None:
            set_(self, "local_shape", _shape2(self.local_shape, "local_shape"))
        if self.shard_axis is not None and self.shard_axis not in {0, 1}:
            raise ValueError("shard_axis must be 0, 1, or None")
        if self.global_scale is not None:
            scale = self.global_scale
            if not isinstance(scale, torch.Tensor) or scale.numel() != 1:
                raise ValueError("global_scale must be a scalar tensor")
            if not bool(torch.isfinite(scale).all()) or bool((scale <= 0).any()):
                raise ValueError("global_scale must be finite and positive")
            set_(self, "global_scale", scale.detach().to(torch.float32).reshape(()))

    @property
    def padding_ratio(self) -> float:
        return float(self.padded_k - self.logical_shape[1]) / float(self.logical_shape[1])

    def to_dict(self) -> dict[str, Any]:
        return {
            "logical_shape": list(self.logical_shape),
            "storage_layout": self.storage_layout,
            "pack_version": self.pack_version,
            "weight_dtype": self.weight_dtype,
            "padded_k": self.padded_k,
            "group_size": self.group_size,
            "packed_bits": self.packed_bits,
            "nibble_order": self.nibble_order,
            "nibble_signed": self.nibble_signed,
            "local_shape": None if self.local_shape is None else list(self.local_shape),
            "shard_axis": self.shard_axis,
            "padding_ratio": self.padding_ratio,
            "global_scale_present": self.global_scale is not None,
            "global_scale_shape": [] if self.global_scale is not None else None,
        }

    @classmethod
    def from_dict(cls, payload: Mapping[str, Any]) -> "PackedWeightMetadata":
        if not isinstance(payload, Mapping):
            raise TypeError("PackedWeightMetadata.from_dict expects a mapping")

        def opt(key: str, cast):
            return None if payload.get(key) is None else cast(payload[key])

        return cls(
            logical_shape=tuple(payload["logical_shape"]),
            storage_layout=str(payload["storage_layout"]),
            pack_version=str(payload["pack_version"]),
            weight_dtype=str(payload["weight_dtype"]),
            padded_k=int(payload["padded_k"]),
            group_size=opt("group_size", int),
            packed_bits=opt("packed_bits", int),
            nibble_order=opt("nibble_order", str),
            nibble_signed=bool(payload.get("nibble_signed", True)),
            local_shape=opt("local_shape", tuple),
            shard_axis=opt("shard_axis", int),
        )


@dataclass(frozen=True, slots=True)
class PackedWeight:
    """Tensor payload + metadata (contracts.py:451-491).  Frozen: never mutated."""

    qweight: Any
    scales: Any | None
    zero_points: Any | None
    metadata: PackedWeightMetadata
    canonical_qweight: Any | None = None
    global_scale: torch.Tensor | None = None
    sparse_mask: torch.Tensor | None = None
    codebook: torch.Tensor | None = None

    def __post_init__(self) -> None:
        if not hasattr(self.qweight, "shape"):
            raise TypeError("PackedWeight.qweight must be a tensor-like object")
        for name in ("scales", "zero_points", "canonical_qweight"):
            value = getattr(self, name)
            if value is not None and not hasattr(value, "shape"):
                raise TypeError(f"PackedWeight.{name} must be tensor-like when provided")
        if self.sparse_mask is not None:
            mask = self.sparse_mask
            if not isinstance(mask, torch.Tensor) or mask.ndim != 2:
                raise TypeError("PackedWeight.sparse_mask must be a rank-2 bool tensor")
            if tuple(mask.shape) != self.metadata.logical_shape:
                raise ValueError("PackedWeight.sparse_mask must match logical_shape")
            if mask.dtype != torch.bool:
                raise TypeError("PackedWeight.sparse_mask must use torch.bool")
        if self.codebook is not None:
            book = self.codebook
            if not isinstance(book, torch.Tensor) or book.ndim != 2:
                raise TypeError("PackedWeight.codebook must be a rank-2 tensor")
            if book.dtype not in {torch.float16, torch.float32, torch.bfloat16}:
                raise TypeError("PackedWeight.codebook must use a floating dtype")

    def to_metadata_dict(self) -> dict[str, Any]:
        return self.metadata.to_dict()


TORCH_DTYPES = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}

__all__ = [
    "EpilogueSpec",
    "GemmProblem",
    "GemmSpec",
    "PackedWeight",
    "PackedWeightMetadata",
    "QuantSpec",
    "TORCH_DTYPES",
]
