"""Runtime module wrappers over the B200 ops, with the surface of xqt's own wrappers.

* :class:`AWQW4A16Linear` -- xqt/runtime/modules/awq_w4a16_linear.py:74-905: owns the execution
  layout of one W4 layer; ``bind`` / ``bind_residual`` hand out hot callables, ``freeze_native_inference``
  drops the canonical copy, ``from_signed_groupwise_storage`` imports xqt's signed group-wise artifact
  (``AWQGPTQWeightOnlyLinear``) through the ``q ^ 0x88``, zero-point-8 bridge (awq_w4a16_linear.py:25-71).
* :class:`B200PackedDequantLinear` -- the operator-stage replacement for a module that exposes xqt's
  duck-typed bridge ``triton_packed_dequant_gemm_args(dtype=, device=)`` (xqt/contracts/weight_only.py:199-224,
  consumed by xqt/kernels/wrappers/triton_dequant_wrappers.py:55-57,144-172): pattern ``gemm_int4_dequant``.
* :class:`Int8MmaLinear` -- xqt/contracts/int8_mma.py:18-343: per-tensor dynamic W8A8.

Every wrapper reports what ran through ``execution_metadata()``, the method xqt's runtime modules and
acceptance reports read (xqt/runtime/modules/composite_add_w4a4.py:304-318).
"""

from __future__ import annotations

from typing import Any, Callable, Iterable

import torch
from torch import nn

from . import native
from .contracts import PackedWeight
from .errors import XQTBackendError
from .layout import signed_storage_to_unsigned
from .ops import awq as awq_ops
from .ops.w4a16 import w4a16_linear

_DTYPE_NAME = {torch.float16: "fp16", torch.bfloat16: "bf16"}
MAX_DECODE_ROWS = 16


class AWQW4A16Linear(nn.Module):
    """Asymmetric group-wise INT4 projection for B200 inference: decode sizes (rows <= 16) on the
    cluster split-K kernel, larger row counts on the tcgen05 GEMM over the canonical bytes."""

    def __init__(self, weight: PackedWeight, *, bias: torch.Tensor | None = None) -> None:
        super().__init__()
        meta = weight.metadata
        self.input_features = int(meta.logical_shape[1])
        self.output_features = int(meta.logical_shape[0])
        self.group_size = int(meta.group_size or 0)
        if bias is not None and bias.numel() != self.output_features:
            raise ValueError("AWQ W4A16 bias size must equal output_features")
        if meta.nibble_signed:
            # signed storage enters through the bridge: u' = s + 8 is byte ^ 0x88, zero point 8
            values = {f: getattr(meta, f) for f in type(meta).__dataclass_fields__}
            values.update(nibble_signed=False)
            weight = PackedWeight(qweight=signed_storage_to_unsigned(weight.qweight), scales=weight.scales,
                                  zero_points=torch.full_like(weight.scales, 8.0), metadata=type(meta)(**values))
        prepacked = awq_ops.prepack_b200_awq_w4a16_decode(weight)
        self._execution_weight = prepacked
        self.register_buffer("qweight", prepacked.qweight)
        self.register_buffer("canonical_qweight", prepacked.canonical_qweight)
        self.register_buffer("weight_scale", prepacked.scales)
        self.register_buffer("weight_zero_point", prepacked.zero_points)
        self.register_buffer("bias", None if bias is None else bias.detach().reshape(-1).to(torch.float32))
        self._has_bias = bias is not None
        self._prepared: dict[torch.dtype, tuple] = {}
        self._bound: dict[tuple[int, torch.dtype], Callable] = {}
        self._residual_bound: dict[tuple[int, torch.dtype], Callable] = {}
        self._native_only = False
        self._native_only_rows: frozenset[int] = frozenset()
        self._native_only_dtype: torch.dtype | None = None
        self._native_only_released_bytes = 0
        self._last_execution: dict[str, Any] = {"implementation": "not_run", "native": False}

    # ------------------------------------------------------------------ construction helpers
    @classmethod
    def from_signed_groupwise_storage(cls, storage: Any, *, device: torch.device | str) -> "AWQW4A16Linear":
        """Build from xqt's signed group-wise artifact (attributes ``quantized_weight`` uint8 ``[N, K/2]``,
        ``weight_scale`` ``[N, G(,1)]``, ``bits``, ``group_size``, ``input_features``, ``output_features``,
        ``padded_input_features``, ``bias``), cf. awq_w4a16_linear.py:25-71,139-153."""

        from .layout import W4_LAYOUT, build_packed_weight
        from .quantize import w4_spec

        bits, group = int(getattr(storage, "bits", 0) or 0), int(getattr(storage, "group_size", 0) or 0)
        n, k = int(getattr(storage, "output_features", 0) or 0), int(getattr(storage, "input_features", 0) or 0)
        qweight, scales = getattr(storage, "quantized_weight", None), getattr(storage, "weight_scale", None)
        if bits != 4 or group not in (64, 128):
            raise XQTBackendError("signed groupwise storage conversion requires 4-bit group-64/128 weights")
        if not isinstance(qweight, torch.Tensor) or qweight.dtype != torch.uint8 or tuple(qweight.shape) != (n, k // 2):
            raise XQTBackendError("signed groupwise storage conversion expects canonical uint8 qweight [N, K/2]")
        if int(getattr(storage, "padded_input_features", k) or k) != k or k % 128:
            raise XQTBackendError("signed groupwise storage conversion needs K == padded K and K % 128 == 0")
        if not isinstance(scales, torch.Tensor):
            raise XQTBackendError("signed groupwise storage conversion expects tensor weight_scale")
        device = torch.device(device)
        scale_2d = scales.reshape(n, k // group).to(device=device, dtype=torch.float32).contiguous()
        spec = w4_spec(group_size=group, symmetric=False)
        weight = build_packed_weight((qweight.detach().to(device) ^ 0x88).contiguous(), logical_shape=(n, k), spec=spec,
                                     scales=scale_2d, zero_points=torch.full_like(scale_2d, 8.0), padded_k=k)
        assert weight.metadata.storage_layout == W4_LAYOUT
        bias = getattr(storage, "bias", None)
        return cls(weight, bias=None if bias is None else bias.to(device))

    # ------------------------------------------------------------------ hot callables
    @property
    def native_only(self) -> bool:
        return self._native_only

    def _parameters_for(self, dtype: torch.dtype):
        hit = self._prepared.get(dtype)
        if hit is None:
            hit = awq_ops.prepare_b200_awq_w4a16_decode_parameters(self._execution_weight, dtype=dtype)
            self._prepared[dtype] = hit
        return hit

    def warmup(self, *, rows: int, dtype: torch.dtype) -> None:
        """Load the library and validate the static contract for this (rows, dtype) outside the hot path."""

        native.library()
        if not awq_ops.native_awq_w4a16_shape_supported(rows, self.input_features, self.output_features, self.group_size):
            raise XQTBackendError(f"AWQ W4A16 decode does not cover rows={rows} for this layer")
        self._parameters_for(dtype)

    def bind(self, *, rows: int, dtype: torch.dtype) -> Callable[[torch.Tensor], torch.Tensor]:
        """Same-shape hot callable with static weights and epilogue state (awq_w4a16_linear.py:605-663)."""

        rows = int(rows)
        if self._native_only and (dtype != self._native_only_dtype or rows not in self._native_only_rows):
            raise RuntimeError(f"native-only AWQ W4A16: rows={rows} / {dtype} were not frozen")
        key = (rows, dtype)
        cached = self._bound.get(key)
        if cached is not None:
            return cached
        self.warmup(rows=rows, dtype=dtype)
        qweight, scales, zeros = self._parameters_for(dtype)
        device = qweight.device
        native_bound = awq_ops.bind_awq_w4a16_decode(
            qweight, scales, zeros, rows=rows, input_features=self.input_features, output_features=self.output_features,
            dtype=dtype, device=device, bias=None if self.bias is None else self.bias.to(device))
        k = self.input_features

        def bound(inputs: torch.Tensor) -> torch.Tensor:
            if inputs.ndim != 2 or tuple(inputs.shape) != (rows, k) or inputs.dtype != dtype or inputs.device != device:
                raise XQTBackendError("bound AWQ W4A16 input disagrees with the static shape/dtype/device")
            return native_bound(inputs)

        self._bound[key] = bound
        return bound

    def bind_residual(self, *, rows: int, dtype: torch.dtype) -> Callable[[torch.Tensor, torch.Tensor], None]:
        """Decode GEMV whose epilogue adds into a residual row in place: ``residual += projection(inputs)``.
        The accumulator is rounded to ``dtype`` before the add, so the result keeps exactly the numerics of
        the unfused ``residual + projection(inputs)`` while one launch disappears (awq_w4a16_linear.py:665-737)."""

        rows = int(rows)
        if self._native_only:
            raise RuntimeError("native-only AWQW4A16Linear cannot bind a residual epilogue")
        if not 1 <= rows <= MAX_DECODE_ROWS:
            raise XQTBackendError(f"bound AWQ W4A16 residual requires 1 <= rows <= {MAX_DECODE_ROWS}")
        if dtype not in _DTYPE_NAME:
            raise XQTBackendError("bound AWQ W4A16 residual requires FP16 or BF16")
        if self.bias is not None:
            raise XQTBackendError("bound AWQ W4A16 residual cannot fold a module bias")
        key = (rows, dtype)
        cached = self._residual_bound.get(key)
        if cached is not None:
            return cached
        self.warmup(rows=rows, dtype=dtype)
        qweight, scales, zeros = self._parameters_for(dtype)
        device, n, k, group = qweight.device, self.output_features, self.input_features, self.group_size
        fn = native.library().xqt_b200_w4a16_decode_lanes
        status = native.status_word(device)
        head = (qweight.data_ptr(), scales.data_ptr(), native.ptr(zeros), 0)
        tail = (rows, n, k, group, 0, native.DTYPE_CODE[dtype], native.DTYPE_CODE[scales.dtype], native.DTYPE_CODE[dtype],
                1, status.data_ptr())     # epilogue flag 1: round the projection before the residual add

        def bound(inputs: torch.Tensor, residual: torch.Tensor) -> None:
            if inputs.ndim != 2 or tuple(inputs.shape) != (rows, k) or inputs.dtype != dtype or inputs.device != device \
                    or not inputs.is_contiguous():
                raise XQTBackendError("bound AWQ W4A16 residual input disagrees with the static shape/dtype/device")
            if residual.ndim != 2 or tuple(residual.shape) != (rows, n) or residual.dtype != dtype or residual.device != device \
                    or not residual.is_contiguous():
                raise XQTBackendError(f"bound AWQ W4A16 residual must be a contiguous [{rows},{n}] {dtype} row")
            code = fn(inputs.data_ptr(), *head, residual.data_ptr(), residual.data_ptr(), *tail,
                      torch.cuda.current_stream(device).cuda_stream)
            if code != 0:
                native.check(code, "xqt_b200_w4a16_decode_lanes")

        bound.keep = (qweight, scales, zeros, status)
        self._residual_bound[key] = bound
        return bound

    def freeze_native_inference(self, *, device: torch.device | str, dtype: torch.dtype, rows: Iterable[int] | int = (1,)) -> int:
        """Irreversibly keep only the execution tensors of the decode path for the given row counts
        (awq_w4a16_linear.py:403-537).  Returns the number of canonical storage bytes released; afterwards
        row counts or dtypes outside the frozen set raise."""

        if self._native_only:
            raise RuntimeError("AWQW4A16Linear is already frozen for native inference")
        if self.training:
            raise RuntimeError("freeze_native_inference requires eval mode")
        if dtype not in _DTYPE_NAME:
            raise ValueError("native-only AWQW4A16Linear requires float16 or bfloat16")
        target = torch.device(device)
        if target.type != "cuda" or self.qweight.device.type != "cuda":
            raise RuntimeError("freeze_native_inference requires CUDA-resident weights")
        frozen = frozenset(int(r) for r in ((rows,) if isinstance(rows, int) else tuple(rows)))
        if not frozen or any(not 1 <= r <= MAX_DECODE_ROWS for r in frozen):
            raise ValueError(f"native-only AWQ W4A16 rows must be between 1 and {MAX_DECODE_ROWS}")
        for r in frozen:
            self.bind(rows=r, dtype=dtype)
        released = self.canonical_qweight.numel() * self.canonical_qweight.element_size()
        self.canonical_qweight = None
        # the execution PackedWeight dropped its canonical bytes too
        self._execution_weight = PackedWeight(qweight=self._execution_weight.qweight, scales=self._execution_weight.scales,
                                              zero_points=self._execution_weight.zero_points,
                                              metadata=self._execution_weight.metadata)
        self._native_only, self._native_only_rows, self._native_only_dtype = True, frozen, dtype
        self._native_only_released_bytes = int(released)
        return int(released)

    # ------------------------------------------------------------------ forward
    def forward(self, inputs: torch.Tensor) -> torch.Tensor:
        if self.training:
            raise RuntimeError("AWQ W4A16 native path requires eval mode")
        if inputs.shape[-1] != self.input_features:
            raise XQTBackendError("AWQ W4A16 input trailing dimension does not match input_features")
        if inputs.dtype not in _DTYPE_NAME:
            raise XQTBackendError("AWQ W4A16 inputs must be float16 or bfloat16")
        flat = inputs.reshape(-1, self.input_features).contiguous()
        rows = int(flat.shape[0])
        if rows <= MAX_DECODE_ROWS and rows >= 1:
            output = self.bind(rows=rows, dtype=flat.dtype)(flat)
            kernel = "w4a16_decode_cl_kernel"
        else:
            if self._native_only:
                raise RuntimeError("native-only AWQ W4A16 serves the frozen decode row counts only")
            output = w4a16_linear(flat, self.canonical_qweight, self.weight_scale, self.weight_zero_point, self.bias,
                                  group_size=self.group_size, nibble_signed=False)
            kernel = "w4a16 tcgen05 GEMM"
        self._last_execution = {
            "implementation": "b200_awq_w4a16", "native": True, "kernel": kernel, "rows": rows,
            "input_features": self.input_features, "output_features": self.output_features, "dtype": _DTYPE_NAME[flat.dtype],
            "bias": self._has_bias, "layout": awq_ops.LANES_LAYOUT,
        }
        return output.reshape(*inputs.shape[:-1], self.output_features)

    def execution_metadata(self) -> dict[str, Any]:
        """Metadata of the most recent invocation plus the frozen-state report."""

        meta = dict(self._last_execution)
        meta.update({
            "native_only": self._native_only, "native_only_rows": sorted(self._native_only_rows),
            "native_only_dtype": None if self._native_only_dtype is None else str(self._native_only_dtype),
            "native_only_released_bytes": self._native_only_released_bytes,
        })
        return meta


class B200PackedDequantLinear(nn.Module):
    """Operator-stage candidate for a weight-only int4 linear: wraps a module that exposes
    ``triton_packed_dequant_gemm_args(dtype=, device=) -> (packed_weight, scale, bias, None, input_features,
    group_size)`` and runs the pattern ``gemm_int4_dequant`` on the B200 kernels.  ``fallback="eager"`` lets
    a non-CUDA input reach the wrapped module's own forward (the operator stage's declared fallback);
    any other value makes that an error."""

    pattern = "gemm_int4_dequant"

    def __init__(self, module: nn.Module, *, fallback: str = "eager", settings: dict | None = None) -> None:
        super().__init__()
        bridge = getattr(module, "triton_packed_dequant_gemm_args", None)
        if not callable(bridge):
            raise XQTBackendError("module does not expose triton_packed_dequant_gemm_args: not a packed int4 linear")
        self.module = module
        self.fallback = str(fallback)
        self.settings = dict(settings or {})
        self._args: dict[tuple, tuple] = {}
        self.last_execution_mode = "not_run"
        self.last_execution_reason: str | None = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from .ops.pattern import gemm_int4_dequant

        if not x.is_cuda:
            if self.fallback != "eager":
                raise XQTBackendError("B200 packed dequant linear needs CUDA tensors and no fallback is configured")
            self.last_execution_mode = "eager_fallback"
            self.last_execution_reason = "input is not a CUDA tensor"
            return self.module(x)
        key = (x.dtype, str(x.device))
        args = self._args.get(key)
        if args is None:
            args = self.module.triton_packed_dequant_gemm_args(dtype=x.dtype, device=x.device)
            self._args[key] = args
        packed_weight, scale, bias, _zero, input_features, group_size = args
        flat = x.reshape(-1, int(input_features))
        activation = getattr(self.module, "activation", None)
        out = gemm_int4_dequant(flat, packed_weight.contiguous(), scale, None, bias, group_size=int(group_size),
                                activation=activation)
        self.last_execution_mode, self.last_execution_reason = "b200_cuda_entry", None
        return out.reshape(*x.shape[:-1], out.shape[-1])

    def execution_metadata(self) -> dict[str, Any]:
        return {
            "engine": "b200_cuda", "operator_family": "linear", "kernel_pattern": self.pattern,
            "execution_mode": self.last_execution_mode, "execution_reason": self.last_execution_reason,
            "weight_source": "weight_only_linear_packed_bridge", "weight_representation": "packed_signed_int4_plus_group_scale",
            "consumes_packed_weight": True, "unpack_stage": "in_kernel", "fallback": self.fallback,
        }


class Int8MmaLinear(nn.Module):
    """xqt's reference W8A8 linear on the B200 tensor cores: per-output-channel int8 weights
    (``qweight_t [K, N]``, ``weight_scale [N]``), ONE dynamic activation scale per call,
    ``scale = max(absmax, eps)/127``, codes clamped to [-127, 127] (xqt/contracts/int8_mma.py:135-149,308-334)."""

    def __init__(self, qweight_t: torch.Tensor, weight_scale: torch.Tensor, bias: torch.Tensor | None = None, *,
                 output_dtype: torch.dtype = torch.bfloat16, eps: float = 1e-6) -> None:
        super().__init__()
        from .ops.w8a8 import pack_convrot_w8a8_linear

        self.input_features, self.output_features = int(qweight_t.shape[0]), int(qweight_t.shape[1])
        self.eps, self.output_dtype = float(eps), output_dtype
        self.register_buffer("qweight_t", qweight_t.to(torch.int8).contiguous())
        self.register_buffer("weight_scale", weight_scale.reshape(-1).to(torch.float32).contiguous())
        self.register_buffer("bias", None if bias is None else bias.detach().reshape(-1).to(torch.float32).contiguous())
        self._packed = None
        self._pack = pack_convrot_w8a8_linear
        self.last_execution: dict[str, Any] = {"engine": "not_run"}

    @classmethod
    def from_linear(cls, module: nn.Linear, *, eps: float = 1e-6) -> "Int8MmaLinear":
        """Per-output-channel symmetric int8 of ``module.weight``: ``scale = max(absmax, eps)/127``."""

        w = module.weight.detach().to(torch.float32)
        scale = (w.abs().amax(dim=1).clamp_min(eps) / 127.0)
        q = torch.round(w / scale.unsqueeze(1)).clamp(-127, 127).to(torch.int8)
        return cls(q.t().contiguous(), scale, module.bias, output_dtype=module.weight.dtype if module.weight.dtype in _DTYPE_NAME
                   else torch.bfloat16, eps=eps)

    def forward(self, inputs: torch.Tensor) -> torch.Tensor:
        from .ops.w8a8 import int8_mma_linear

        if inputs.shape[-1] != self.input_features:
            raise XQTBackendError("Int8MmaLinear input trailing dimension does not match input_features")
        if self._packed is None or self._packed.qweight.device != inputs.device or self._packed.dtype != inputs.dtype:
            self._packed = self._pack(self.qweight_t.to(inputs.device), self.weight_scale.to(inputs.device),
                                      None if self.bias is None else self.bias.to(inputs.device), dtype=inputs.dtype)
        out = int8_mma_linear(inputs, self._packed, eps=self.eps)
        self.last_execution = {
            "engine": "b200_cuda", "true_int8_mma": True, "activation_dtype": "int8", "weight_dtype": "int8",
            "accumulation_dtype": "int32", "activation_scale_mode": "dynamic", "activation_granularity": "per_tensor",
            "input_rows": int(inputs.numel() // self.input_features), "input_features": self.input_features,
            "output_features": self.output_features,
        }
        return out

    def execution_metadata(self) -> dict[str, Any]:
        return dict(self.last_execution)


__all__ = ["AWQW4A16Linear", "B200PackedDequantLinear", "Int8MmaLinear", "MAX_DECODE_ROWS"]
