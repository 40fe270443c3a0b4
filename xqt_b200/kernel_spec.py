"""Kernel namespace: op x backend table, capability filtering, fixed-path selection.

Torch-free mirror of xqt's unified kernel namespace (xqt/kernels/spec.py:15-194,
xqt/kernels/registry.py:11-79, xqt/kernels/selector.py:39-95,196-202): ``KernelSpec(op, backend,
target="module:attr", capabilities)`` with a lazy ``load()``, ``register_kernel`` that raises on a
conflicting (op, backend) pair, ``select_kernel`` honouring ``XQT_FORCE_BACKEND`` and device
capability, ``get_kernel``.  The rows registered at the bottom are this backend's: the same op names
xqt registers for its sm_89 kernels (xqt/kernels/ops/quantization/__init__.py:104-176), backend
``custom_cuda``, capability window sm_100 only.
"""

from __future__ import annotations

import importlib
import os
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, FrozenSet, Optional, Tuple

from .errors import XQTBackendError


class KernelBackend(str, Enum):
    TORCH = "torch"
    TRITON = "triton"
    TILELANG = "tilelang"
    CUTLASS = "cutlass"
    CUTE_DSL = "cute_dsl"
    CUSTOM_CUDA = "custom_cuda"
    TVM_FFI = "tvm_ffi"


class DeviceType(str, Enum):
    CUDA = "cuda"
    CPU = "cpu"


@dataclass(frozen=True, slots=True)
class PlatformInfo:
    device_type: str = "cpu"
    cuda_arch_major: Optional[int] = None
    cuda_arch_minor: Optional[int] = None

    @property
    def device(self) -> DeviceType:
        return DeviceType.CUDA if self.device_type == "cuda" else DeviceType.CPU

    @classmethod
    def detect(cls) -> "PlatformInfo":
        try:
            import torch

            if torch.cuda.is_available():
                major, minor = torch.cuda.get_device_capability()
                return cls("cuda", major, minor)
        except Exception:  # noqa: BLE001
            pass
        return cls()


@dataclass(frozen=True, slots=True)
class CapabilityRequirement:
    device: DeviceType
    min_cuda_arch: Optional[Tuple[int, int]] = None
    max_cuda_arch: Optional[Tuple[int, int]] = None

    @classmethod
    def cuda(cls, min_sm: Optional[Tuple[int, int]] = None, max_sm: Optional[Tuple[int, int]] = None):
        return cls(DeviceType.CUDA, min_sm, max_sm)

    def is_satisfied_by(self, platform: PlatformInfo) -> bool:
        """Same device kind, and -- for CUDA with a known compute capability -- inside the
        inclusive ``[min_cuda_arch, max_cuda_arch]`` window (an open end is unbounded)."""

        if platform.device != self.device:
            return False
        if self.device != DeviceType.CUDA or platform.cuda_arch_major is None:
            return True
        have = (platform.cuda_arch_major, platform.cuda_arch_minor or 0)
        low = self.min_cuda_arch if self.min_cuda_arch is not None else have
        high = self.max_cuda_arch if self.max_cuda_arch is not None else have
        return low <= have <= high


@dataclass(frozen=True, slots=True)
class KernelSpec:
    op: str
    backend: KernelBackend
    target: str
    capabilities: FrozenSet[CapabilityRequirement] = field(default_factory=frozenset)
    description: str = ""

    @property
    def group(self) -> str:
        return self.op.split(".", 1)[0]

    @property
    def name(self) -> str:
        return self.op.split(".", 1)[1] if "." in self.op else self.op

    def is_available(self, platform: PlatformInfo) -> bool:
        return not self.capabilities or any(c.is_satisfied_by(platform) for c in self.capabilities)

    def load(self) -> Callable[..., object]:
        if ":" not in self.target:
            raise XQTBackendError(f"invalid kernel target {self.target!r} for op {self.op!r}")
        module_name, attr_path = self.target.split(":", 1)
        try:
            obj: object = importlib.import_module(module_name)
        except ImportError as exc:
            raise XQTBackendError(f"kernel backend {self.backend.value!r} for op {self.op!r} not available: {exc}") from exc
        try:
            for part in attr_path.split("."):
                obj = getattr(obj, part)
        except AttributeError as exc:
            raise XQTBackendError(f"kernel target {self.target!r} not found for op {self.op!r}: {exc}") from exc
        if not callable(obj):
            raise XQTBackendError(f"kernel target {self.target!r} for op {self.op!r} is not callable")
        return obj  # type: ignore[return-value]


class KernelRegistry:
    def __init__(self) -> None:
        self._by_op: dict[str, list[KernelSpec]] = {}

    def register(self, spec: KernelSpec) -> KernelSpec:
        existing = self._by_op.setdefault(spec.op, [])
        for other in existing:
            if other.backend == spec.backend:
                if other != spec:
                    raise ValueError(
                        f"Conflicting kernel registration for op {spec.op!r}, backend {spec.backend.value!r}: "
                        f"{other.target!r} != {spec.target!r}")
                return spec
        existing.append(spec)
        return spec

    def get(self, op: str) -> list[KernelSpec]:
        return list(self._by_op.get(op, ()))

    def ops(self) -> list[str]:
        return sorted(self._by_op)

    def clear(self) -> None:
        self._by_op.clear()


registry = KernelRegistry()


def register_kernel(spec: KernelSpec) -> KernelSpec:
    return registry.register(spec)


def select_kernel(op: str, backend: Optional[KernelBackend] = None, *, platform: Optional[PlatformInfo] = None,
                  table: Optional[KernelRegistry] = None) -> KernelSpec:
    specs = (table or registry).get(op)
    if not specs:
        raise KeyError(f"No kernels registered for op {op!r}")
    forced = os.environ.get("XQT_FORCE_BACKEND", "").strip().lower()
    if backend is None and forced:
        backend = next((s.backend for s in specs if s.backend.value == forced), None)
    if backend is not None:
        for spec in specs:
            if spec.backend == backend:
                return spec
        raise KeyError(f"No '{backend.value}' backend registered for op {op!r}")
    if len(specs) == 1:
        return specs[0]
    platform = platform or PlatformInfo.detect()
    eligible = [s for s in specs if s.is_available(platform)]
    if len(eligible) == 1:
        return eligible[0]
    if not eligible:
        raise ValueError(f"op {op!r} has no backend usable on device {platform.device.value!r} "
                         f"(registered: {[s.backend.value for s in specs]})")
    raise ValueError(f"op {op!r} has multiple backends usable on device {platform.device.value!r} "
                     f"({[s.backend.value for s in eligible]}); pass backend=... to choose one")


def get_kernel(op: str, backend: Optional[KernelBackend] = None) -> Callable[..., object]:
    return select_kernel(op, backend).load()


SM100 = frozenset({CapabilityRequirement.cuda(min_sm=(10, 0), max_sm=(10, 0))})

B200_KERNELS = (
    KernelSpec("quantization.awq_w4a16_decode", KernelBackend.CUSTOM_CUDA, "xqt_b200.ops.awq:awq_w4a16_decode", SM100,
               "AWQ W4A16 decode (M<=16), xqt's signature: cluster split-K kernel on the lane-ordered layout"),
    KernelSpec("quantization.awq_w4a8_decode", KernelBackend.CUSTOM_CUDA, "xqt_b200.ops.awq:awq_w4a8_decode", SM100,
               "AWQ W4A8 decode (M<=16): int8 activation codes as exact integers through the cluster decode kernel"),
    KernelSpec("quantization.w4a16_decode_tiled", KernelBackend.CUSTOM_CUDA, "xqt_b200.ops.w4a16:w4a16_decode_tiled", SM100,
               "W4A16 decode (M<=16) on a TiledW4 execution layout (lanes / rows128 / tile128)"),
    KernelSpec("quantization.w4a16_linear", KernelBackend.CUSTOM_CUDA, "xqt_b200.ops.w4a16:w4a16_linear", SM100,
               "W4A16 linear on canonical xqt_int4_nk_v1 tensors, any M"),
    KernelSpec("quantization.convrot_w8a8_linear", KernelBackend.CUSTOM_CUDA, "xqt_b200.ops.w8a8:convrot_w8a8_linear", SM100,
               "ConvRot W8A8 linear: rotation + per-token int8 + tcgen05 kind::i8 GEMM"),
    KernelSpec("quantization.svdq_w4a4_linear", KernelBackend.CUSTOM_CUDA, "xqt_b200.ops.w4a4:svdq_w4a4_linear", SM100,
               "SVDQuant W4A4 linear with rank-r branch"),
    KernelSpec("quantization.svdq_w8a8_linear", KernelBackend.CUSTOM_CUDA, "xqt_b200.ops.svdq_w8a8:svdq_w8a8_linear", SM100,
               "SVDQuant W8A8 linear: per-token int8 (scale in the activation dtype) x per-channel int8 + rank-r branch"),
    KernelSpec("quantization.convrot_w4a4_rowwise_linear", KernelBackend.CUSTOM_CUDA,
               "xqt_b200.ops.w4a4:convrot_w4a4_linear", SM100, "ConvRot W4A4 linear (no low-rank branch)"),
    KernelSpec("quantization.gemm_int4_dequant", KernelBackend.CUSTOM_CUDA, "xqt_b200.ops.pattern:gemm_int4_dequant", SM100,
               "operator-stage W4 pattern: signed nibbles, w = scale * code - zero (zero in real units)"),
    KernelSpec("quantization.int8_mma_linear", KernelBackend.CUSTOM_CUDA, "xqt_b200.ops.w8a8:int8_mma_linear", SM100,
               "per-tensor dynamic W8A8 (Int8MmaLinear semantics) on tcgen05 kind::i8"),
    KernelSpec("quantization.swiglu", KernelBackend.CUSTOM_CUDA, "xqt_b200.ops.mlp:swiglu", SM100, "fused SwiGLU gating"),
)
for _spec in B200_KERNELS:
    register_kernel(_spec)

__all__ = ["B200_KERNELS", "CapabilityRequirement", "DeviceType", "KernelBackend", "KernelRegistry",
           "KernelSpec", "PlatformInfo", "SM100", "get_kernel", "register_kernel", "registry", "select_kernel"]
