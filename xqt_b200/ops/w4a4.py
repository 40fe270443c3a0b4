"""W4A4 SVDQuant / ConvRot linear on B200.

Python surface of xqt's native op (xqt/kernels/ops/_impl/cute/svdq_w4a4_sm89.py:379-557,963-1318):
``pack_svdq_w4a4_linear`` -> ``PackedSVDQW4A4Linear``, ``svdq_w4a4_linear(inputs, packed,
workspace=None, lora_scale=1.0)``, ``bind_svdq_w4a4_linear``, ``convrot_w4a4_linear`` (no low-rank
branch).  The packed contents are backend-private: here the weight stays in the composite artifact's
own canonical signed-nibble bytes (``packed_residual``, xqt/contracts/composite.py:92-227) -- the
artifact's integer codes are consumed as they are, not re-quantised from a dequantised copy as the
sm_89 path does (xqt/runtime/modules/composite_add_w4a4.py:198-216) -- plus a small per-tile block of
transposed scales and up factors.

Per call: rotate + round + group-64 int4 quantisation (one kernel), rank-R down projection (one
kernel), then one of two forms of the product.  Integer form (M < 256): tcgen05 ``kind::i8`` GEMM with
per-slab fp32 scaling, rank-R up projection and bias in the epilogue.  Operand-dequantised form
(``form="dense"``, opt-in): both operands expanded once to fp16 (code x scale), the low-rank pair
appended along K, one dense tcgen05 fp16 GEMM -- the per-group scaling of the integer form runs on the
CUDA cores and bounds it well below the tensor peak.  Codes and scales are identical in both forms;
the dense form's fp16 operand rounding costs accuracy (rel-L2 1.2e-3 at K = 3072 against the 1e-3 bar),
which is why it is not the default.
"""

from __future__ import annotations

from dataclasses import dataclass, replace

import torch

from .. import native
from ..errors import XQTBackendError
from ..quantize import Rotation, quantize_residual_int4
from .activation import rotate_quantize

GROUP = 64
RANK_PAD = 32
TILE = 128


@dataclass(frozen=True)
class PackedSVDQW4A4Linear:
    qweight: torch.Tensor          # uint8 [N, K/2] canonical signed nibbles
    aux: torch.Tensor              # fp32 [ceil(N/128), K/64*128 + 128*32]
    weight_scales: torch.Tensor    # fp32 [N, K/64]: the artifact's residual_scale (read by the dense form)
    up: torch.Tensor | None        # fp32 [N, 32] up factors, rank padded with zeros (None without low-rank branch)
    down: torch.Tensor             # dtype [32, K], rows past the rank are zero
    bias: torch.Tensor | None      # fp32 [N]
    input_features: int
    output_features: int
    padded_input_features: int
    rank: int
    dtype: torch.dtype
    rotation: Rotation | None = None
    act_granularity: str = "group"     # "group": one scale per (token, 64 K); "token": one per token (ConvRot artifact form)
    weight_bytes: torch.Tensor | None = None   # uint8 [N, K]: operand cache of `with_operand_cache` (None: widened per call)

    @property
    def padded_rank(self) -> int:
        return RANK_PAD


def _operand_image(values: torch.Tensor) -> torch.Tensor:
    """fp32 ``[rows (a multiple of 128), 32]`` -> fp32-typed view of the tensor-core operand image: per row bf16
    ``[hi(32) | lo(32)]`` (``hi = bf16(v)``, ``lo = bf16(v - hi)``), its eight 16-byte chunks at index ``c ^ (row & 7)``."""

    rows = int(values.shape[0])
    hi = values.to(torch.bfloat16)
    lo = (values - hi.to(torch.float32)).to(torch.bfloat16)
    chunks = torch.cat((hi, lo), dim=1).reshape(rows, 8, 8)                     # 8 chunks of 8 bf16
    index = torch.arange(8, device=values.device).reshape(1, 8) ^ (torch.arange(rows, device=values.device).reshape(rows, 1) & 7)
    image = torch.gather(chunks, 1, index.reshape(rows, 8, 1).expand(rows, 8, 8))   # physical chunk c holds logical chunk c ^ (row & 7)
    return image.contiguous().view(torch.float32).reshape(rows, RANK_PAD)


def pack_svdq_w4a4_linear(
    residual_weight: torch.Tensor | None,
    down_weight: torch.Tensor | None,
    up_weight: torch.Tensor | None,
    bias: torch.Tensor | None = None,
    *,
    smooth: torch.Tensor | None = None,
    norm_weight: torch.Tensor | None = None,
    packed_residual: torch.Tensor | None = None,
    residual_scale: torch.Tensor | None = None,
    dtype: torch.dtype = torch.bfloat16,
    rotation: Rotation | None = None,
    device: torch.device | None = None,
    act_granularity: str = "group",
) -> PackedSVDQW4A4Linear:
    """Build the B200 layout.  Pass the artifact's ``packed_residual`` / ``residual_scale``
    (group 64) to keep its integer codes bit for bit; otherwise ``residual_weight`` ``[N,K]`` is
    quantised with the artifact's own rule (scale = absmax/7, xqt/compression/quant/quantizers/svd.py:92-128).
    ``down_weight`` is ``[r,K]``, ``up_weight`` ``[N,r]`` (None for a layer without low-rank branch)."""

    if act_granularity not in ("group", "token"):
        raise XQTBackendError("act_granularity must be 'group' (per token and 64 K) or 'token'")
    if smooth is not None or norm_weight is not None:
        # xqt's sm_89 kernel can divide the activation by a per-channel smoothing vector and fuse an
        # RMSNorm weight into its quantise prologue (svdq_w4a4_sm89.py:471-557); neither is served here
        raise XQTBackendError("SVDQ W4A4 on B200 does not serve smooth / norm_weight prologues")
    if packed_residual is None:
        if residual_weight is None:
            raise XQTBackendError("pack_svdq_w4a4_linear needs residual_weight or packed_residual")
        packed_residual, residual_scale, _ = quantize_residual_int4(residual_weight, group_size=GROUP)
    if residual_scale is None:
        raise XQTBackendError("packed_residual needs its residual_scale")
    if dtype not in (torch.float16, torch.bfloat16):
        raise XQTBackendError("SVDQ W4A4 supports fp16 or bf16 activations")
    device = packed_residual.device if device is None else device
    n, k = int(packed_residual.shape[0]), int(packed_residual.shape[1]) * 2
    groups = k // GROUP
    if packed_residual.dtype != torch.uint8 or tuple(residual_scale.shape) != (n, groups):
        raise XQTBackendError(f"SVDQ W4A4 residual must be uint8 [N,K/2] with group-64 scales [{n},{groups}]")
    if not native.library().xqt_b200_w4a4_supported(1, n, k):
        raise XQTBackendError("SVDQ W4A4 on B200 needs K % 128 == 0 and N % 8 == 0")
    rank = 0 if down_weight is None else int(down_weight.shape[0])
    if rank > RANK_PAD:
        raise XQTBackendError(f"SVDQ W4A4 on B200 supports rank <= {RANK_PAD}")
    if (down_weight is None) != (up_weight is None):
        raise XQTBackendError("down_weight and up_weight come together")
    tiles = -(-n // TILE)
    scale = residual_scale.to(device=device, dtype=torch.float32)
    sw = torch.zeros((tiles * TILE, groups), device=device, dtype=torch.float32)
    sw[:n] = scale * float(2 ** 18)           # both operands reach the tensor core as code * 2^-9 (FP8 E4M3 bytes)
    up = torch.zeros((tiles * TILE, RANK_PAD), device=device, dtype=torch.float32)
    down = torch.zeros((RANK_PAD, k), device=device, dtype=dtype)
    if rank:
        if tuple(down_weight.shape) != (rank, k) or tuple(up_weight.shape) != (n, rank):
            raise XQTBackendError("low-rank factors must be down [r,K] and up [N,r]")
        up[:n, :rank] = up_weight.to(device=device, dtype=dtype).to(torch.float32)
        down[:rank] = down_weight.to(device=device, dtype=dtype)
    aux = torch.cat((sw.reshape(tiles, TILE, groups).transpose(1, 2).reshape(tiles, -1),
                     _operand_image(up).reshape(tiles, -1)), dim=1).contiguous()
    return PackedSVDQW4A4Linear(
        qweight=packed_residual.to(device).contiguous(), aux=aux, weight_scales=scale.contiguous(),
        up=up[:n].contiguous() if rank else None, down=down,
        bias=None if bias is None else bias.reshape(-1).to(device=device, dtype=torch.float32).contiguous(),
        input_features=k, output_features=n, padded_input_features=k, rank=rank, dtype=dtype, rotation=rotation,
        act_granularity=act_granularity)


@dataclass
class W4A4Workspace:
    """Per-call scratch of the linear (field names of xqt's, svdq_w4a4_sm89.py:399-409): activation codes
    ``[rows, K]`` (int4 values in int8), their scales ``[rows, K/64]``, the low-rank activation
    ``[ceil(rows/128)*128, 32]`` fp32, plus the rotated activation the low-rank branch reads."""

    quantized_activation: torch.Tensor
    activation_scales: torch.Tensor
    lora_activation: torch.Tensor | None = None
    row_scales: torch.Tensor | None = None
    rotated_activation: torch.Tensor | None = None

    @property
    def padded_rows(self) -> int:
        return int(self.quantized_activation.shape[0])


def allocate_w4a4_workspace(rows: int, packed: PackedSVDQW4A4Linear, *, with_lora_rank: int = 0,
                            with_row_scales: bool = False) -> W4A4Workspace:
    """Scratch for calls of up to ``rows`` rows (cf. svdq_w4a4_sm89.py:963-1000).  ``with_lora_rank`` > 0
    adds the buffers of the low-rank branch (any rank up to 32 uses the padded width 32)."""

    if with_row_scales:
        raise XQTBackendError("row-wise activation scales are not served by the B200 W4A4 kernels")
    if int(with_lora_rank) > RANK_PAD:
        raise XQTBackendError(f"SVDQ W4A4 on B200 supports rank <= {RANK_PAD}")
    rows, k, device = int(rows), packed.padded_input_features, packed.qweight.device
    lora = None
    rotated = torch.empty((rows, k), dtype=packed.dtype, device=device)
    if int(with_lora_rank) > 0:
        lora = torch.zeros((-(-rows // TILE) * TILE, RANK_PAD), dtype=torch.float32, device=device)
    return W4A4Workspace(
        quantized_activation=torch.empty((rows, k), dtype=torch.int8, device=device),
        activation_scales=torch.empty((-(-rows // TILE) * TILE, k // GROUP), dtype=torch.float32, device=device),   # room for the tile-major order
        lora_activation=lora, rotated_activation=rotated)


def native_w4a4_available(*, build: bool = False) -> bool:
    """Whether the B200 W4A4 backend can run on the current device (cf. svdq_w4a4_sm89.py:152-168)."""

    import os

    if not torch.cuda.is_available() or torch.cuda.get_device_capability() != (10, 0):
        return False
    if os.environ.get("XQT_DISABLE_B200", "0") not in {"", "0"}:
        return False
    return native.available() if build else native.LIBRARY_PATH.exists()


def native_w4a4_shape_supported(input_features: int, output_features: int) -> bool:
    try:
        return bool(native.library().xqt_b200_w4a4_supported(1, int(output_features), int(input_features)))
    except Exception:  # noqa: BLE001 - a missing library means "not supported"
        return False


def native_convrot_w4a4_shape_supported(logical_input_features: int, rotated_input_features: int, output_features: int,
                                        rot_size: int) -> bool:
    size = int(rot_size)
    return (0 < int(logical_input_features) <= int(rotated_input_features) and size >= 1 and (size & (size - 1)) == 0
            and int(rotated_input_features) % max(size, GROUP) == 0
            and native_w4a4_shape_supported(rotated_input_features, output_features))


def native_w4a4_version() -> str:
    return native.version()


def svdq_w4a4_linear(inputs: torch.Tensor, packed: PackedSVDQW4A4Linear, *, workspace: W4A4Workspace | None = None, lora_scale: float = 1.0,
                     return_parts: bool = False, form: str = "auto"):
    """Full forward: rotation (``packed.rotation``; None = input already rotated), int4 activations
    per (token, 64-K), GEMM with per-group scales, low-rank branch, bias.  ``form``: ``integer``
    (tcgen05 int8 MMA, per-group int32 sums scaled in fp32), ``dense`` (operands expanded to fp16 once,
    dense fp16 MMA, faster from M = 256, rel-L2 up to 1.2e-3) or ``auto`` (the integer form)."""

    if inputs.shape[-1] != packed.input_features or inputs.dtype != packed.dtype:
        raise XQTBackendError("SVDQ W4A4 input trailing dimension or dtype does not match the packed layer")
    x = inputs.reshape(-1, packed.input_features).contiguous()
    m, k, n = int(x.shape[0]), packed.input_features, packed.output_features
    device = x.device
    out = torch.empty((m, n), device=device, dtype=packed.dtype)
    if m == 0:
        return out.reshape(*inputs.shape[:-1], n)
    lib = native.library()
    buffers = None
    if workspace is not None:
        if workspace.padded_rows < m or int(workspace.quantized_activation.shape[1]) != k \
                or workspace.rotated_activation is None or (packed.rank and workspace.lora_activation is None):
            raise ValueError("workspace extent does not match inputs / packed weights")
        buffers = (workspace.quantized_activation, workspace.activation_scales, workspace.rotated_activation)
    dense = form == "dense"
    if form not in ("auto", "dense", "integer"):
        raise XQTBackendError("form must be auto, dense or integer")
    # The integer form's GEMM takes the codes as sign-magnitude bytes (FP8 E4M3 operands), the dense form as int8.
    # direct: the prologue kernels write the GEMM's own operand forms (tile-major scales, low-rank operand images), so
    # the GEMM call launches no preparation kernel; callers that want the parts back, or scale the low-rank
    # activations, take the row-major forms.
    direct = not dense and not return_parts and lora_scale == 1.0
    codes, scales, rotated = rotate_quantize(x, packed.rotation, bits=4, group_size=GROUP if packed.act_granularity == "group" else 0,
                                             return_rotated=True, out=buffers, sign_magnitude=not dense, tiled_scales=direct)
    if workspace is not None and workspace.lora_activation is not None:
        la = workspace.lora_activation          # rows past M stay zero: the kernels only write rows < M
    elif direct and packed.rank:
        la = torch.empty((-(-m // TILE) * TILE, RANK_PAD), device=device, dtype=torch.float32)   # holds the operand images
    else:
        la = torch.zeros((-(-m // TILE) * TILE, RANK_PAD), device=device, dtype=torch.float32)
    # flags 1 | 2: scales tile-major, la holds operand images (without a low-rank branch la is all zero bits, which is
    # a zero image as well as a zero matrix)
    flags = 3 if direct else 0
    stream = native.stream_handle(device)
    # auto keeps the integer form: it is the one that meets the 1e-3 parity bar at every K (the dense
    # form is about 3.5x faster at M >= 256 and within 1.2e-3)
    with torch.cuda.device(device):
        scratch = native.workspace(device, lib.xqt_b200_w4a4_dense_workspace_bytes(m, n, k) if dense else
                                   lib.xqt_b200_w4a4_workspace_bytes(m, n, k), "gemm")
        if packed.rank:
            if dense:
                native.check(lib.xqt_b200_lowrank_down_tc(
                    rotated.data_ptr(), packed.down.data_ptr(), la.data_ptr(), m, k, native.DTYPE_CODE[packed.dtype],
                    scratch.data_ptr(), scratch.numel(), stream), "xqt_b200_lowrank_down_tc")
            else:
                native.check(lib.xqt_b200_lowrank_down(rotated.data_ptr(), packed.down.data_ptr(), 0 if direct else la.data_ptr(),
                                                       la.data_ptr() if direct else 0, m, k,
                                                       native.DTYPE_CODE[packed.dtype], stream), "xqt_b200_lowrank_down")
            if lora_scale != 1.0:
                la[:m].mul_(float(lora_scale))
        if dense:
            native.check(lib.xqt_b200_w4a4_dense(
                codes.data_ptr(), scales.data_ptr(), packed.qweight.data_ptr(), packed.weight_scales.data_ptr(),
                la.data_ptr() if packed.rank else 0, native.ptr(packed.up), native.ptr(packed.bias), out.data_ptr(), m, n, k,
                native.DTYPE_CODE[packed.dtype], scratch.data_ptr(), scratch.numel(), stream), "xqt_b200_w4a4_dense")
        else:
            native.check(lib.xqt_b200_w4a4_gemm(
                codes.data_ptr(), scales.data_ptr(), packed.qweight.data_ptr(), native.ptr(packed.weight_bytes), packed.aux.data_ptr(), la.data_ptr(),
                native.ptr(packed.bias), out.data_ptr(), m, n, k, native.DTYPE_CODE[packed.dtype], flags, scratch.data_ptr(),
                scratch.numel(), stream), "xqt_b200_w4a4_gemm")
    out = out.reshape(*inputs.shape[:-1], n)
    if return_parts:
        from .activation import decode_sign_magnitude

        return out, {"codes": codes if dense else decode_sign_magnitude(codes), "scales": scales, "rotated": rotated, "la": la[:m]}
    return out


def convrot_w4a4_linear(inputs: torch.Tensor, packed: PackedSVDQW4A4Linear, *, rot_size: int | None = None,
                        workspace: W4A4Workspace | None = None) -> torch.Tensor:
    """ConvRot W4A4 (no low-rank branch): same kernels with an empty rank-R term
    (cf. svdq_w4a4_sm89.py:1082-1100).  A layer packed with ``act_granularity="token"`` reproduces the
    artifact's own per-token activation scale (``ConvRotMixedPrecisionLinear``, convrot_4bit.py:669-679,
    what its row-wise native kernel computes)."""

    if rot_size is not None and packed.rotation is not None and int(rot_size) != packed.rotation.block:
        raise XQTBackendError("rot_size disagrees with the rotation the layer was packed with")
    return svdq_w4a4_linear(inputs, packed, workspace=workspace)


def with_operand_cache(packed: PackedSVDQW4A4Linear) -> PackedSVDQW4A4Linear:
    """The layer with its weights also held in the GEMM's operand form (one sign-magnitude byte per weight, ``[N, K]``
    uint8 beside the packed half byte): the integer form then skips its per-call widening pass.  A memory-for-time
    choice of the caller; the packed storage stays the layer's definition."""

    if packed.weight_bytes is not None:
        return packed
    n, k, device = packed.output_features, packed.input_features, packed.qweight.device
    widened = torch.empty((n, k), dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        native.check(native.library().xqt_b200_w4a4_expand_weight(packed.qweight.data_ptr(), widened.data_ptr(), n, k,
                                                                   native.stream_handle(device)), "xqt_b200_w4a4_expand_weight")
    return replace(packed, weight_bytes=widened)


def bind_svdq_w4a4_linear(packed: PackedSVDQW4A4Linear, workspace: W4A4Workspace | None = None, *, rows: int,
                          lora_scale: float = 1.0, operand_cache: bool = False):
    """Validated state for the steady-state path (cf. svdq_w4a4_sm89.py:1264-1318): the workspace owns the
    codes, scales, rotated activation and low-rank activation, so a call allocates only its output.
    ``operand_cache``: hold the weights in operand form as well (see ``with_operand_cache``)."""

    rows = int(rows)
    if operand_cache:
        packed = with_operand_cache(packed)
    if workspace is None:
        workspace = allocate_w4a4_workspace(rows, packed, with_lora_rank=packed.rank)
    if workspace.padded_rows < rows or (packed.rank and workspace.lora_activation is None):
        raise ValueError("SVDQuant workspace does not match rows / rank")
    k, dtype, device = packed.input_features, packed.dtype, packed.qweight.device

    def run(inputs: torch.Tensor) -> torch.Tensor:
        if inputs.dtype != dtype or inputs.device != device or inputs.shape[-1] != k or inputs.numel() != rows * k:
            raise XQTBackendError("bound SVDQ W4A4 call: input shape, dtype or device mismatch")
        return svdq_w4a4_linear(inputs, packed, workspace=workspace, lora_scale=lora_scale)

    run.keep = (packed, workspace)
    return run


__all__ = ["PackedSVDQW4A4Linear", "W4A4Workspace", "allocate_w4a4_workspace", "bind_svdq_w4a4_linear", "convrot_w4a4_linear",
           "native_convrot_w4a4_shape_supported", "native_w4a4_available", "native_w4a4_shape_supported", "native_w4a4_version",
           "pack_svdq_w4a4_linear", "svdq_w4a4_linear", "with_operand_cache"]
