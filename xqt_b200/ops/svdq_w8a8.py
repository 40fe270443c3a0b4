"""SVDQuant W8A8 on B200: int8 x int8 GEMM with a rank-R low-rank branch, under the names of xqt's native op
(xqt/kernels/ops/_impl/cute/svdq_w8a8_sm89.py): ``pack_svdq_w8a8_linear``, ``allocate_svdq_w8a8_workspace``,
``svdq_w8a8_linear``, ``bind_svdq_w8a8_linear``, ``w8a8_linear`` and the ``native_svdq_w8a8_*`` probes.

    s_a[m] = T(amax_m / 127),  q_a = clamp(rint(x / s_a))          rotate_quant kernel, mode 9 (no rotation)
    la     = x down^T            (fp32 [M, 32])                      lowrank_down_kernel
    low    = T(lora_scale la) up^T   (fp32 [M, N])                   dense tcgen05 GEMM, bf16/fp16 operands
    y      = T(int32(q_a q_w^T) s_a s_w + bias + low)                gemm_i8_kernel, fp32 addend in the epilogue

The reference's kernels are svdq_w8a8_sm89_kernel.cu (quantize_act_lora / gemm_lora); it multiplies by approximate
reciprocals of the scales where this path divides (IEEE), which can move a code that sits on a rounding boundary."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import native
from ..errors import XQTBackendError
from .activation import rotate_quantize

RANK_PAD = 32          # the down projection's width
UP_PAD = 64            # the up projection's K extent (one 64-element tensor-core K block)


@dataclass(frozen=True)
class PackedSVDQW8A8Linear:
    qweight: torch.Tensor          # int8 [N, K]
    weight_scales: torch.Tensor    # fp32 [N] (values representable in the activation dtype)
    bias: torch.Tensor | None      # fp32 [N]
    down: torch.Tensor             # dtype [32, K], rows past the rank are zero
    up: torch.Tensor               # dtype [N, 64], columns past the rank are zero
    input_features: int
    output_features: int
    rank: int
    dtype: torch.dtype

    @property
    def padded_rank(self) -> int:
        return RANK_PAD


@dataclass
class W8A8SVDQWorkspace:
    quantized_activation: torch.Tensor     # int8 [rows, K]
    activation_scales: torch.Tensor        # fp32 [rows]
    lora_activation: torch.Tensor          # fp32 [rows, 32]
    lora_activation16: torch.Tensor        # dtype [rows, 64], columns past 32 stay zero
    low_rank_output: torch.Tensor          # fp32 [rows, N]

    @property
    def padded_rows(self) -> int:
        return int(self.quantized_activation.shape[0])


def native_svdq_w8a8_shape_supported(input_features: int, output_features: int, rank: int) -> bool:
    """K a multiple of 32 (the down projection's K step), N a multiple of 8, rank <= 32."""

    return int(input_features) > 0 and int(input_features) % 32 == 0 and int(output_features) > 0 \
        and int(output_features) % 8 == 0 and 0 <= int(rank) <= RANK_PAD


def native_svdq_w8a8_available(*, build: bool = False) -> bool:
    if not torch.cuda.is_available() or torch.cuda.get_device_capability() != (10, 0):
        return False
    return native.available() if build else native.LIBRARY_PATH.exists()


def native_svdq_w8a8_version() -> str:
    return native.version()


def pack_svdq_w8a8_linear(residual_weight: torch.Tensor, down_weight: torch.Tensor | None, up_weight: torch.Tensor | None,
                          bias: torch.Tensor | None = None) -> PackedSVDQW8A8Linear:
    """Per-output-channel int8 weights with ``scale = T(absmax/127)`` (1 for a zero row), as the reference's pack
    (svdq_w8a8_sm89.py:158-232); ``down_weight`` ``[rank, K]``, ``up_weight`` ``[N, rank]`` in the weight's dtype."""

    if residual_weight.ndim != 2 or residual_weight.dtype not in (torch.bfloat16, torch.float16) or not residual_weight.is_cuda:
        raise XQTBackendError("SVDQ W8A8: residual_weight must be a CUDA bf16/fp16 [N, K] tensor")
    n, k = (int(v) for v in residual_weight.shape)
    rank = 0 if down_weight is None else int(down_weight.shape[0])
    if not native_svdq_w8a8_shape_supported(k, n, rank):
        raise XQTBackendError("SVDQ W8A8 on B200 requires K % 32 == 0, N % 8 == 0 and rank <= 32")
    dtype, device = residual_weight.dtype, residual_weight.device
    if rank and (tuple(down_weight.shape) != (rank, k) or up_weight is None or tuple(up_weight.shape) != (n, rank)):
        raise ValueError("down_weight must be [rank, K] and up_weight [N, rank]")
    w = residual_weight.to(torch.float32)
    amax = w.abs().amax(dim=1)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax)).to(dtype).to(torch.float32)
    q = torch.round(w / scale[:, None]).clamp_(-128, 127).to(torch.int8).contiguous()
    down = torch.zeros((RANK_PAD, k), device=device, dtype=dtype)
    up = torch.zeros((n, UP_PAD), device=device, dtype=dtype)
    if rank:
        down[:rank] = down_weight.to(device=device, dtype=dtype)
        up[:, :rank] = up_weight.to(device=device, dtype=dtype)
    if bias is not None and (bias.ndim != 1 or int(bias.numel()) != n):
        raise ValueError("bias must match output_features")
    return PackedSVDQW8A8Linear(
        qweight=q, weight_scales=scale.contiguous(),
        bias=None if bias is None else bias.to(device=device, dtype=torch.float32).contiguous(),
        down=down, up=up, input_features=k, output_features=n, rank=rank, dtype=dtype)


def allocate_svdq_w8a8_workspace(rows: int, packed: PackedSVDQW8A8Linear) -> W8A8SVDQWorkspace:
    rows, k, n, device = int(rows), packed.input_features, packed.output_features, packed.qweight.device
    return W8A8SVDQWorkspace(
        quantized_activation=torch.empty((rows, k), dtype=torch.int8, device=device),
        activation_scales=torch.empty((rows,), dtype=torch.float32, device=device),
        lora_activation=torch.empty((rows, RANK_PAD), dtype=torch.float32, device=device),
        lora_activation16=torch.zeros((rows, UP_PAD), dtype=packed.dtype, device=device),
        low_rank_output=torch.empty((rows, n), dtype=torch.float32, device=device))


def _forward(inputs: torch.Tensor, packed: PackedSVDQW8A8Linear, workspace: W8A8SVDQWorkspace | None, lora_scale: float,
             low_rank: bool, return_parts: bool = False):
    if inputs.ndim != 2 or inputs.dtype != packed.dtype or not inputs.is_cuda:
        raise XQTBackendError("SVDQ W8A8: inputs must be a CUDA rank-2 tensor in the packed layer's dtype")
    if int(inputs.shape[1]) != packed.input_features:
        raise ValueError("inputs do not match packed input_features")
    if inputs.device != packed.qweight.device:
        raise XQTBackendError("inputs and packed weights must share a CUDA device")
    x = inputs.contiguous()
    m, k, n, device = int(x.shape[0]), packed.input_features, packed.output_features, x.device
    out = torch.empty((m, n), dtype=packed.dtype, device=device)
    if m == 0:
        return out
    ws = workspace or allocate_svdq_w8a8_workspace(m, packed)
    if ws.padded_rows < m or int(ws.quantized_activation.shape[1]) != k or int(ws.low_rank_output.shape[1]) != n:
        raise ValueError("workspace extent does not match inputs")
    codes, scales = rotate_quantize(x, None, bits=8, out=(ws.quantized_activation, ws.activation_scales), scale_in_act_dtype=True)
    lib, stream, dcode = native.library(), native.stream_handle(device), native.DTYPE_CODE[packed.dtype]
    low_ptr = 0
    with torch.cuda.device(device):
        scratch = native.workspace(device, 256, "gemm")
        if low_rank and packed.rank:
            la, la16, low = ws.lora_activation[:m], ws.lora_activation16[:m], ws.low_rank_output[:m]
            native.check(lib.xqt_b200_lowrank_down(x.data_ptr(), packed.down.data_ptr(), la.data_ptr(), 0, m, k, dcode, stream),
                         "xqt_b200_lowrank_down")
            if lora_scale != 1.0:
                la.mul_(float(lora_scale))
            la16[:, :RANK_PAD].copy_(la)                     # the rounding to the activation dtype
            native.check(lib.xqt_b200_lowrank_up(la16.data_ptr(), packed.up.data_ptr(), low.data_ptr(), m, n, UP_PAD, dcode,
                                                 scratch.data_ptr(), scratch.numel(), stream), "xqt_b200_lowrank_up")
            low_ptr = low.data_ptr()
        native.check(lib.xqt_b200_w8a8_gemm_addend(
            codes.data_ptr(), packed.qweight.data_ptr(), scales.data_ptr(), packed.weight_scales.data_ptr(), native.ptr(packed.bias),
            low_ptr, out.data_ptr(), m, n, k, dcode, scratch.data_ptr(), scratch.numel(), stream), "xqt_b200_w8a8_gemm_addend")
    if return_parts:
        return out, {"codes": codes, "scales": scales}
    return out


def svdq_w8a8_linear(inputs: torch.Tensor, packed: PackedSVDQW8A8Linear, *, workspace: W8A8SVDQWorkspace | None = None,
                     lora_scale: float = 1.0, return_parts: bool = False):
    """Dynamic per-token int8 activations x per-channel int8 weights + low-rank branch (svdq_w8a8_sm89.py:258-312)."""

    return _forward(inputs, packed, workspace, float(lora_scale), True, return_parts)


def w8a8_linear(inputs: torch.Tensor, packed: PackedSVDQW8A8Linear, *, workspace: W8A8SVDQWorkspace | None = None) -> torch.Tensor:
    """The same dynamic W8A8 path without the low-rank branch (svdq_w8a8_sm89.py:380-425)."""

    return _forward(inputs, packed, workspace, 1.0, False)


def bind_svdq_w8a8_linear(packed: PackedSVDQW8A8Linear, workspace: W8A8SVDQWorkspace | None = None, *, rows: int,
                          lora_scale: float = 1.0):
    """Validated state for the steady-state path (svdq_w8a8_sm89.py:314-377): the workspace is fixed here, a call
    allocates only its output."""

    rows = int(rows)
    if workspace is None:
        workspace = allocate_svdq_w8a8_workspace(rows, packed)
    if workspace.padded_rows < rows:
        raise ValueError("workspace row extent does not match rows")
    k, n, dtype, device, scale = packed.input_features, packed.output_features, packed.dtype, packed.qweight.device, float(lora_scale)
    # every pointer and code of the library calls is resolved here; a call checks its input, allocates its output and
    # makes the calls (the general entry's per-call validation costs more host time than the kernels run)
    lib, dcode = native.library(), native.DTYPE_CODE[dtype]
    index = device.index if device.index is not None else torch.cuda.current_device()
    codes, scales = workspace.quantized_activation[:rows], workspace.activation_scales[:rows]
    la, la16, low = workspace.lora_activation[:rows], workspace.lora_activation16[:rows], workspace.low_rank_output[:rows]
    la16_head = la16[:, :RANK_PAD]
    scratch = native.workspace(device, 256, "gemm")
    quant_tail = (0, codes.data_ptr(), scales.data_ptr(), 0, rows, k, 0, 0, 9, 0, dcode)
    down_args = (packed.down.data_ptr(), la.data_ptr(), 0, rows, k, dcode)
    up_args = (la16.data_ptr(), packed.up.data_ptr(), low.data_ptr(), rows, n, UP_PAD, dcode, scratch.data_ptr(), scratch.numel())
    gemm_head = (codes.data_ptr(), packed.qweight.data_ptr(), scales.data_ptr(), packed.weight_scales.data_ptr(), native.ptr(packed.bias),
                 low.data_ptr() if packed.rank else 0)
    gemm_tail = (rows, n, k, dcode, scratch.data_ptr(), scratch.numel())
    has_rank = bool(packed.rank)

    def run(inputs: torch.Tensor) -> torch.Tensor:
        if inputs.dtype != dtype or inputs.device != device or inputs.ndim != 2 or tuple(inputs.shape) != (rows, k) \
                or not inputs.is_contiguous():
            raise XQTBackendError("bound SVDQ W8A8 call: input shape, dtype, device or layout mismatch")
        if torch.cuda.current_device() != index:
            raise XQTBackendError("bound SVDQ W8A8 call: make the weight's device current before calling")
        out = torch.empty((rows, n), device=device, dtype=dtype)
        stream = torch.cuda.current_stream(device).cuda_stream
        x_ptr = inputs.data_ptr()
        code = lib.xqt_b200_rotate_quantize(x_ptr, *quant_tail, stream)
        if code == 0 and has_rank:
            code = lib.xqt_b200_lowrank_down(x_ptr, *down_args, stream)
            if code == 0:
                if scale != 1.0:
                    la.mul_(scale)
                la16_head.copy_(la)                          # the rounding to the activation dtype
                code = lib.xqt_b200_lowrank_up(*up_args, stream)
        if code == 0:
            code = lib.xqt_b200_w8a8_gemm_addend(*gemm_head, out.data_ptr(), *gemm_tail, stream)
        if code != 0:
            native.check(code, "bound SVDQ W8A8 (quantise / low-rank / GEMM)")
        return out

    run.keep = (packed, workspace, scratch)
    return run


__all__ = ["PackedSVDQW8A8Linear", "W8A8SVDQWorkspace", "allocate_svdq_w8a8_workspace", "bind_svdq_w8a8_linear",
           "native_svdq_w8a8_available", "native_svdq_w8a8_shape_supported", "native_svdq_w8a8_version",
           "pack_svdq_w8a8_linear", "svdq_w8a8_linear", "w8a8_linear"]
