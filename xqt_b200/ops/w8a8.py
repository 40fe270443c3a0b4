"""ConvRot-style W8A8 int8 linear on B200.

Python surface of xqt's native op (xqt/kernels/ops/_impl/cute/convrot_w8a8_sm89.py:154-500):
``pack_convrot_w8a8_linear`` -> ``PackedConvRotW8A8Linear``; ``convrot_w8a8_linear(inputs, packed,
rotated_input_features=..., rot_size=...)``; ``bind_convrot_w8a8_linear``.  The packed tensor
contents are backend-private; here the weight is simply int8 ``[N, K]`` K-major (what the TMA
descriptor of the tcgen05 GEMM reads), produced from the artifact's transposed ``qweight_t [K, N]``
(xqt/compression/quant/quantizers/convrot_int8.py:361-400).

Per call: one prologue kernel (rotate, round to the activation dtype, per-token int8) and one
tcgen05 ``kind::i8`` GEMM whose epilogue applies ``a_scale[m] * w_scale[n]`` (+ bias) in fp32.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import native
from ..errors import XQTBackendError
from ..quantize import Rotation, regular_rotation
from .activation import rotate_quantize


@dataclass(frozen=True)
class PackedConvRotW8A8Linear:
    qweight: torch.Tensor          # int8 [N, padded_K], K-major
    weight_scales: torch.Tensor    # fp32 [N]
    bias: torch.Tensor | None      # fp32 [N]
    input_features: int
    output_features: int
    padded_input_features: int
    dtype: torch.dtype


def pack_convrot_w8a8_linear(qweight_t: torch.Tensor, weight_scale: torch.Tensor, bias: torch.Tensor | None = None,
                             *, dtype: torch.dtype = torch.bfloat16,
                             input_features: int | None = None) -> PackedConvRotW8A8Linear:
    """``qweight_t`` is the artifact's int8 ``[padded_K, N]`` buffer, ``weight_scale`` its fp32 ``[N]``."""

    if qweight_t.ndim != 2 or qweight_t.dtype != torch.int8:
        raise XQTBackendError("ConvRot W8A8 qweight_t must be int8 [K, N]")
    if dtype not in (torch.float16, torch.bfloat16):
        raise XQTBackendError("ConvRot W8A8 supports fp16 or bf16 activations")
    kp, n = int(qweight_t.shape[0]), int(qweight_t.shape[1])
    if weight_scale.numel() != n:
        raise XQTBackendError("ConvRot W8A8 weight_scale must have N elements")
    if kp % 16 or n % 8:
        raise XQTBackendError("ConvRot W8A8 on B200 needs padded K % 16 == 0 and N % 8 == 0")
    device = qweight_t.device
    return PackedConvRotW8A8Linear(
        qweight=qweight_t.t().contiguous(), weight_scales=weight_scale.reshape(-1).to(torch.float32).contiguous(),
        bias=None if bias is None else bias.reshape(-1).to(device=device, dtype=torch.float32).contiguous(),
        input_features=kp if input_features is None else int(input_features), output_features=n,
        padded_input_features=kp, dtype=dtype)


def w8a8_gemm(codes: torch.Tensor, act_scale: torch.Tensor, packed: PackedConvRotW8A8Linear,
              out: torch.Tensor | None = None) -> torch.Tensor:
    m, k = int(codes.shape[0]), int(codes.shape[1])
    n = packed.output_features
    device = codes.device
    if codes.dtype != torch.int8 or k != packed.padded_input_features or not codes.is_contiguous():
        raise XQTBackendError("W8A8 GEMM: activation codes must be contiguous int8 [M, padded_K]")
    if packed.qweight.device != device:
        raise XQTBackendError("W8A8 GEMM: weight and activation must share a device")
    if out is None:
        out = torch.empty((m, n), device=device, dtype=packed.dtype)
    if m == 0:
        return out
    scratch = native.workspace(device, 256, "gemm")
    with torch.cuda.device(device):
        code = native.library().xqt_b200_w8a8_gemm(
            codes.data_ptr(), packed.qweight.data_ptr(), act_scale.data_ptr(), packed.weight_scales.data_ptr(),
            native.ptr(packed.bias), out.data_ptr(), m, n, k, native.DTYPE_CODE[packed.dtype], scratch.data_ptr(),
            scratch.numel(), native.stream_handle(device))
    native.check(code, "xqt_b200_w8a8_gemm")
    return out


def int8_mma_linear(inputs: torch.Tensor, packed: PackedConvRotW8A8Linear, *, eps: float = 1e-6) -> torch.Tensor:
    """xqt's reference W8A8 linear ``Int8MmaLinear`` on the tensor cores (xqt/contracts/int8_mma.py:308-334):
    one dynamic activation scale for the whole tensor, ``scale = max(absmax, eps)/127``, codes clamped to
    [-127, 127], no rotation; ``out = int32(q_a q_w^T) * (a_scale * w_scale[n]) + bias``.  ``packed`` comes from
    :func:`pack_convrot_w8a8_linear` (the module's ``qweight_t`` / ``weight_scale`` buffers)."""

    from .activation import quantize_int8_per_tensor

    if inputs.dtype != packed.dtype or not inputs.is_cuda or inputs.device != packed.qweight.device:
        raise XQTBackendError("Int8MmaLinear inputs must match the packed layer's dtype and device")
    if inputs.shape[-1] != packed.input_features or packed.padded_input_features != packed.input_features:
        raise XQTBackendError("Int8MmaLinear input trailing dimension does not match input_features")
    x = inputs.reshape(-1, packed.input_features)
    codes, row_scales, _ = quantize_int8_per_tensor(x, eps=eps)
    return w8a8_gemm(codes, row_scales, packed).reshape(*inputs.shape[:-1], packed.output_features)


def _rms_norm(flat: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    x = flat.to(torch.float32)
    return (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight.to(torch.float32)).to(flat.dtype)


class SharedConvRotW8A8Group:
    """Projections that share one rotated, quantised activation (cf. convrot_w8a8_sm89.py:601-661): the
    rotate + quantise prologue runs once, one GEMM per projection.  ``norm_weight`` (RMSNorm ahead of the
    projections) is applied by an eager fp32 pass here, not inside the prologue kernel."""

    def __init__(self, packeds: list, *, rot_size: int = 256, norm_weight: torch.Tensor | None = None, eps: float = 1e-6) -> None:
        if not packeds:
            raise ValueError("packeds must contain at least one projection")
        first = packeds[0]
        if any((p.input_features, p.padded_input_features, p.dtype, p.qweight.device) !=
               (first.input_features, first.padded_input_features, first.dtype, first.qweight.device) for p in packeds):
            raise XQTBackendError("grouped ConvRot W8A8 projections must share input size, dtype and device")
        self.packeds, self.rot_size = list(packeds), int(rot_size)
        self.input_features, self.padded_input_features = first.input_features, first.padded_input_features
        self.dtype, self.device = first.dtype, first.qweight.device
        self.norm_weight = None if norm_weight is None else norm_weight.to(device=self.device, dtype=self.dtype)
        self.eps = float(eps)
        self._rotation = None if self.rot_size == 1 else regular_rotation(self.rot_size)

    def _quantise(self, inputs: torch.Tensor):
        flat = inputs.reshape(-1, self.input_features)
        if flat.dtype != self.dtype or flat.device != self.device:
            raise XQTBackendError("grouped ConvRot W8A8 inputs must match the packed layers' dtype and device")
        if self.norm_weight is not None:
            flat = _rms_norm(flat, self.norm_weight, self.eps)
        if self.padded_input_features != self.input_features:
            flat = torch.nn.functional.pad(flat, (0, self.padded_input_features - self.input_features))
        return rotate_quantize(flat.contiguous(), self._rotation, bits=8)

    def __call__(self, inputs: torch.Tensor) -> list:
        codes, scales = self._quantise(inputs)
        return [w8a8_gemm(codes, scales, p).reshape(*inputs.shape[:-1], p.output_features) for p in self.packeds]


class FusedConvRotW8A8LinearGroup(SharedConvRotW8A8Group):
    """The same group as ONE horizontal GEMM over the concatenated output channels
    (cf. convrot_w8a8_sm89.py:664-917): one prologue, one tcgen05 GEMM, the outputs are column slices of its
    result.  ``forward_swiglu`` (two projections, gate then up) feeds the fused result to the SwiGLU kernel.
    The reference's small-row fallbacks to a dense de-quantised GEMM are not needed: the int8 GEMM serves every M."""

    def __init__(self, packeds: list, *, rot_size: int = 256, norm_weight: torch.Tensor | None = None, eps: float = 1e-6,
                 min_int8_rows: int = 0) -> None:
        super().__init__(packeds, rot_size=rot_size, norm_weight=norm_weight, eps=eps)
        self.split_sizes = [p.output_features for p in self.packeds]
        self.total_output_features = sum(self.split_sizes)
        self.min_int8_rows = int(min_int8_rows)         # accepted for signature parity; unused
        bias = None
        if any(p.bias is not None for p in self.packeds):
            bias = torch.cat([p.bias if p.bias is not None else torch.zeros(p.output_features, device=self.device) for p in self.packeds])
        self.fused_packed = PackedConvRotW8A8Linear(
            qweight=torch.cat([p.qweight for p in self.packeds], dim=0).contiguous(),
            weight_scales=torch.cat([p.weight_scales for p in self.packeds]).contiguous(), bias=bias,
            input_features=self.input_features, output_features=self.total_output_features,
            padded_input_features=self.padded_input_features, dtype=self.dtype)

    def _fused(self, inputs: torch.Tensor) -> torch.Tensor:
        codes, scales = self._quantise(inputs)
        return w8a8_gemm(codes, scales, self.fused_packed)

    def __call__(self, inputs: torch.Tensor) -> list:
        fused = self._fused(inputs)
        return [part.reshape(*inputs.shape[:-1], part.shape[-1]) for part in torch.split(fused, self.split_sizes, dim=1)]

    def forward_swiglu(self, inputs: torch.Tensor) -> torch.Tensor:
        """``silu(gate(x)) * up(x)`` from the fused gate|up GEMM and the SwiGLU kernel."""

        from .mlp import swiglu

        if len(self.packeds) != 2 or self.split_sizes[0] != self.split_sizes[1]:
            raise XQTBackendError("forward_swiglu requires exactly two packed projections (gate and up) of equal width")
        out = swiglu(self._fused(inputs))
        return out.reshape(*inputs.shape[:-1], self.split_sizes[0])



_REGULAR_SIZES = (1, 4, 16, 64, 256, 1024)


def native_convrot_w8a8_available(dtype: torch.dtype, *, build: bool = False) -> bool:
    """Whether the B200 W8A8 backend can run on the current device (cf. convrot_w8a8_sm89.py:128-149)."""

    import os

    if dtype not in (torch.float16, torch.bfloat16):
        return False
    if not torch.cuda.is_available() or torch.cuda.get_device_capability() != (10, 0):
        return False
    if os.environ.get("XQT_DISABLE_B200", "0") not in {"", "0"}:
        return False
    return native.available() if build else native.LIBRARY_PATH.exists()


def native_convrot_w8a8_shape_supported(logical_input_features: int, rotated_input_features: int, output_features: int,
                                        rot_size: int) -> bool:
    """Same predicate shape as xqt's (convrot_w8a8_sm89.py:35-50); the B200 kernels take every regular
    Hadamard order up to 1024 (xqt: 256 only), K a multiple of 16 and N a multiple of 8."""

    logical_k, rotated_k = int(logical_input_features), int(rotated_input_features)
    return (0 < logical_k <= rotated_k and int(output_features) > 0 and int(output_features) % 8 == 0
            and int(rot_size) in _REGULAR_SIZES and rotated_k % max(int(rot_size), 16) == 0)


def native_prerotated_w8a8_shape_supported(rotated_input_features: int, output_features: int) -> bool:
    return int(rotated_input_features) > 0 and int(rotated_input_features) % 16 == 0 and int(output_features) > 0 \
        and int(output_features) % 8 == 0


def native_convrot_w8a8_version(dtype: torch.dtype) -> str:
    del dtype
    return native.version()


@dataclass
class ConvRotW8A8Workspace:
    """Per-call scratch of the linear (cf. convrot_w8a8_sm89.py:168-176): int8 activation codes
    ``[rows, padded K]`` and their per-token scales ``[rows]``."""

    quantized_activation: torch.Tensor
    activation_scales: torch.Tensor

    @property
    def padded_rows(self) -> int:
        return int(self.quantized_activation.shape[0])


def allocate_convrot_w8a8_workspace(rows: int, packed: PackedConvRotW8A8Linear) -> ConvRotW8A8Workspace:
    device = packed.qweight.device
    return ConvRotW8A8Workspace(
        quantized_activation=torch.empty((int(rows), packed.padded_input_features), dtype=torch.int8, device=device),
        activation_scales=torch.empty((int(rows),), dtype=torch.float32, device=device))


def convrot_w8a8_linear(inputs: torch.Tensor, packed: PackedConvRotW8A8Linear, *,
                        rotated_input_features: int | None = None, rot_size: int = 256,
                        workspace: ConvRotW8A8Workspace | None = None, rotation: Rotation | None = None) -> torch.Tensor:
    """Full forward, signature of xqt's op (convrot_w8a8_sm89.py:365-372).

    ``rotated_input_features`` is the (padded) K the weight was rotated and quantised at; it must equal
    ``packed.input_features`` (default).  ``rot_size`` is the regular Hadamard block; ``rot_size == 1``
    means the caller already rotated the input (rounding and quantisation still happen).  ``rotation``
    (an extension) supplies a non-regular rotation, e.g. a seeded Sylvester block.  With a ``workspace``
    of at least the call's rows the prologue allocates nothing."""

    if inputs.dtype != packed.dtype:
        raise XQTBackendError("inputs must match the packed ConvRot W8A8 dtype")
    if not inputs.is_cuda or inputs.device != packed.qweight.device:
        raise XQTBackendError("inputs and packed weights must share a CUDA device")
    rotated_k = packed.input_features if rotated_input_features is None else int(rotated_input_features)
    if isinstance(rotated_input_features, bool) or rotated_k != packed.input_features:
        raise XQTBackendError("native ConvRot W8A8 shape or rotation size is unsupported: rotated_input_features "
                              "must be the K the layer was packed with")
    logical_k = int(inputs.shape[-1])
    if rotation is None:
        supported = native_prerotated_w8a8_shape_supported(rotated_k, packed.output_features) if int(rot_size) == 1 else \
            native_convrot_w8a8_shape_supported(logical_k, rotated_k, packed.output_features, int(rot_size))
        if not supported:
            raise XQTBackendError("native ConvRot W8A8 shape or rotation size is unsupported")
    if logical_k > rotated_k:
        raise XQTBackendError("ConvRot W8A8 input trailing dimension exceeds rotated_input_features")
    x = inputs.reshape(-1, logical_k)
    pad = packed.padded_input_features - logical_k
    if pad:
        x = torch.nn.functional.pad(x, (0, pad))
    rot = rotation if rotation is not None else (None if int(rot_size) == 1 else regular_rotation(int(rot_size)))
    out_buffers = None
    if workspace is not None:
        if workspace.padded_rows < x.shape[0] or int(workspace.quantized_activation.shape[1]) != packed.padded_input_features:
            raise ValueError("workspace extent does not match inputs / packed weights")
        out_buffers = (workspace.quantized_activation, workspace.activation_scales)
    codes, scales = rotate_quantize(x, rot, bits=8, out=out_buffers)
    out = w8a8_gemm(codes, scales, packed)
    return out.reshape(*inputs.shape[:-1], packed.output_features)


def bind_convrot_w8a8_linear(packed: PackedConvRotW8A8Linear, workspace: ConvRotW8A8Workspace | None = None, *, rows: int,
                             rotated_input_features: int | None = None, rot_size: int = 256,
                             rotation: Rotation | None = None):
    """Validated state for the steady-state path (cf. convrot_w8a8_sm89.py:441-500): shapes, rotation
    vector and scratch are fixed here; the callable makes the two library calls (prologue, GEMM) and
    allocates only its output."""

    rows = int(rows)
    rotated_k = packed.input_features if rotated_input_features is None else int(rotated_input_features)
    if rotated_k != packed.input_features or packed.padded_input_features != packed.input_features:
        raise XQTBackendError("bound ConvRot W8A8: rotated_input_features must be the (unpadded) K of the packed layer")
    if workspace is None:
        workspace = allocate_convrot_w8a8_workspace(rows, packed)
    if workspace.padded_rows < rows or int(workspace.quantized_activation.shape[1]) != packed.padded_input_features:
        raise ValueError("workspace extent does not match rows / packed weights")
    rot = rotation if rotation is not None else (None if int(rot_size) == 1 else regular_rotation(int(rot_size)))
    device, k, n, dtype = packed.qweight.device, packed.input_features, packed.output_features, packed.dtype
    if k % (1 if rot is None else rot.block):
        raise XQTBackendError("the rotated dimension must be a multiple of the rotation block")
    # every pointer and code of the two library calls is resolved here; a call checks its input, allocates its output
    # and makes the two calls (the general entry's per-call validation costs about as much host time as the kernels run)
    from .activation import _KIND, _column_scale

    lib = native.library()
    codes, scales = workspace.quantized_activation[:rows], workspace.activation_scales[:rows]
    column_scale = None if rot is None else _column_scale(rot, device)
    index = device.index if device.index is not None else torch.cuda.current_device()
    scratch = native.workspace(device, 256, "gemm")
    dcode = native.DTYPE_CODE[dtype]
    prologue = (native.ptr(column_scale), codes.data_ptr(), scales.data_ptr(), 0, rows, k, _KIND[None if rot is None else rot.kind],
                0 if rot is None else rot.block, 8, 0, dcode)
    gemm_head = (codes.data_ptr(), packed.qweight.data_ptr(), scales.data_ptr(), packed.weight_scales.data_ptr(), native.ptr(packed.bias))
    gemm_tail = (rows, n, k, dcode, scratch.data_ptr(), scratch.numel())

    def run(inputs: torch.Tensor) -> torch.Tensor:
        if inputs.dtype != dtype or inputs.device != device or inputs.shape[-1] != k or inputs.numel() != rows * k \
                or not inputs.is_contiguous():
            raise XQTBackendError("bound ConvRot W8A8 call: input shape, dtype, device or layout mismatch")
        if torch.cuda.current_device() != index:
            raise XQTBackendError("bound ConvRot W8A8 call: make the weight's device current before calling")
        out = torch.empty((*inputs.shape[:-1], n), device=device, dtype=dtype)
        stream = torch.cuda.current_stream(device).cuda_stream
        code = lib.xqt_b200_rotate_quantize(inputs.data_ptr(), *prologue, stream)
        if code == 0:
            code = lib.xqt_b200_w8a8_gemm(*gemm_head, out.data_ptr(), *gemm_tail, stream)
        if code != 0:
            native.check(code, "bound ConvRot W8A8 (xqt_b200_rotate_quantize / xqt_b200_w8a8_gemm)")
        return out

    run.keep = (packed, workspace, rot, column_scale, scratch)
    return run


__all__ = ["ConvRotW8A8Workspace", "FusedConvRotW8A8LinearGroup", "PackedConvRotW8A8Linear", "SharedConvRotW8A8Group", "allocate_convrot_w8a8_workspace", "bind_convrot_w8a8_linear",
           "convrot_w8a8_linear", "int8_mma_linear", "native_convrot_w8a8_available", "native_convrot_w8a8_shape_supported",
           "native_convrot_w8a8_version", "native_prerotated_w8a8_shape_supported", "pack_convrot_w8a8_linear", "w8a8_gemm"]
