"""Canonical packed-weight layouts of the quantized-linear path.

The byte layouts here are the cross-backend storage contract and must not change:

* ``xqt_int4_nk_v1`` (xqt/kernels/ops/gemm/layout.py:80-109,571-585,786-867):
  ``qweight`` is ``uint8 [N, ceil(padded_K/2)]``; byte ``j`` of row ``n`` holds
  ``k = 2j`` in its low nibble and ``k = 2j+1`` in its high nibble.  Signed
  weights store two's-complement nibbles, unsigned weights store codes 0..15
  and carry ``zero_points``.  ``scales`` / ``zero_points`` are ``[N, G]`` with
  ``G = padded_K / group_size`` and ``group_size`` in {32, 64, 128}.
* ``xqt_int8_nk_v1``: ``int8 [N, K]`` with per-channel scales ``[N, 1]``.

Everything in this file is host logic on torch tensors (CPU or CUDA, no custom
kernels); the B200-specific execution layouts are derived from these by
:mod:`xqt_b200.prepack` and are private to this backend.
"""

from __future__ import annotations

import torch

from .contracts import PackedWeight, PackedWeightMetadata, QuantSpec

W4_LAYOUT = "xqt_int4_nk_v1"
W8_LAYOUT = "xqt_int8_nk_v1"
_INT_DTYPES = {torch.uint8, torch.int8, torch.int16, torch.int32, torch.int64}
# HF AutoAWQ stores the eight nibbles of an int32 word in this order
# (layout.py:234-239): nibble position p of the word is logical element order[p].
AWQ_NIBBLE_ORDER = (0, 4, 1, 5, 2, 6, 3, 7)


def _pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    if codes.shape[1] % 2:
        codes = torch.nn.functional.pad(codes, (0, 1), value=0)
    codes = codes.to(torch.uint8)
    return (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()


def pack_int4_signed(values: torch.Tensor) -> torch.Tensor:
    """Signed values in [-8, 7] -> canonical bytes, low nibble first (layout.py:80-93)."""

    if values.ndim != 2:
        raise ValueError("INT4 values must be rank-2 [N,K]")
    if values.dtype not in _INT_DTYPES - {torch.uint8}:
        raise TypeError("INT4 values must use an integer dtype")
    wide = values.to(torch.int16)
    if bool(((wide < -8) | (wide > 7)).any()):
        raise ValueError("signed INT4 values must be in [-8, 7]")
    return _pack_nibbles(wide & 0x0F)


def pack_int4_unsigned(values: torch.Tensor) -> torch.Tensor:
    """Unsigned codes in [0, 15] -> canonical bytes, low nibble first (layout.py:96-109)."""

    if values.ndim != 2:
        raise ValueError("INT4 values must be rank-2 [N,K]")
    if values.dtype not in _INT_DTYPES:
        raise TypeError("INT4 values must use an integer dtype")
    wide = values.to(torch.int16)
    if bool(((wide < 0) | (wide > 15)).any()):
        raise ValueError("unsigned INT4 values must be in [0, 15]")
    return _pack_nibbles(wide)


def unpack_int4(packed: torch.Tensor, *, logical_k: int, signed: bool) -> torch.Tensor:
    """Inverse of the two packers: int8 values when signed, uint8 codes otherwise (layout.py:571-585)."""

    if packed.ndim != 2 or packed.dtype != torch.uint8:
        raise TypeError("packed INT4 weights must be uint8 rank-2")
    k = int(logical_k)
    if k <= 0 or packed.shape[1] < (k + 1) // 2:
        raise ValueError("logical_k is incompatible with packed INT4 shape")
    codes = torch.stack((packed & 0x0F, packed >> 4), dim=-1).reshape(packed.shape[0], -1)[:, :k]
    if not signed:
        return codes.contiguous()
    wide = codes.to(torch.int16)
    return (wide - ((wide & 8) << 1)).to(torch.int8)


def unpack_int4_signed(packed: torch.Tensor, *, logical_k: int) -> torch.Tensor:
    return unpack_int4(packed, logical_k=logical_k, signed=True)


def expected_weight_scale_shape(
    logical_shape: tuple[int, int], *, granularity: str, group_size: int | None = None
) -> tuple[int, ...]:
    """Canonical scale shape for a ``[N,K]`` weight (layout.py:43-60)."""

    n, k = int(logical_shape[0]), int(logical_shape[1])
    if granularity == "per_tensor":
        return (1, 1)
    if granularity == "per_channel":
        return (n, 1)
    if granularity in {"groupwise", "blockwise"}:
        if group_size is None or int(group_size) <= 0:
            raise ValueError("groupwise/blockwise scales require group_size > 0")
        return (n, -(-k // int(group_size)))
    raise ValueError(f"unsupported weight scale granularity: {granularity!r}")


def _check_scale(value, *, shape: tuple[int, int], spec: QuantSpec, name: str) -> None:
    if value is None:
        raise ValueError(f"{name} is required for quantized packed weights")
    expected = expected_weight_scale_shape(
        shape, granularity=spec.weight_granularity, group_size=spec.group_size
    )
    actual = tuple(int(item) for item in value.shape)
    if actual == expected:
        return
    if spec.weight_granularity == "per_channel" and actual == (shape[0],):
        return
    if spec.weight_granularity == "per_tensor" and actual in {(), (1,)}:
        return
    raise ValueError(f"{name} expected shape {expected}, got {actual}")


def build_packed_weight(
    qweight: torch.Tensor,
    *,
    logical_shape: tuple[int, int],
    spec: QuantSpec,
    scales: torch.Tensor | None,
    zero_points: torch.Tensor | None = None,
    padded_k: int | None = None,
    storage_layout: str | None = None,
    pack_version: str | None = None,
    local_shape: tuple[int, int] | None = None,
    shard_axis: int | None = None,
) -> PackedWeight:
    """Wrap already-quantized tensors without touching their values (layout.py:635-783).

    Only the dtypes of this path (int4, int8 and dense) are accepted.
    """

    n, k = int(logical_shape[0]), int(logical_shape[1])
    if qweight.ndim != 2 or int(qweight.shape[0]) != n:
        raise ValueError("qweight must have shape [N, packed-or-logical-K]")
    padded = k if padded_k is None else int(padded_k)
    if spec.weight_dtype == "int4":
        columns = (padded + 1) // 2
        if int(qweight.shape[1]) != columns:
            raise ValueError(f"packed 4-bit qweight must have {columns} columns, got {qweight.shape[1]}")
        packed_bits, nibble_order = 4, "low_high"
    elif spec.weight_dtype in {"int8", "fp16", "bf16", "fp32"}:
        if int(qweight.shape[1]) != padded:
            raise ValueError("non-INT4 qweight must use padded logical K columns")
        packed_bits, nibble_order = None, None
    else:
        raise ValueError(f"weight dtype {spec.weight_dtype!r} is outside the quantized-linear path")
    if spec.weight_dtype in {"int4", "int8"}:
        _check_scale(scales, shape=(n, padded), spec=spec, name="scales")
        if zero_points is not None:
            _check_scale(zero_points, shape=(n, padded), spec=spec, name="zero_points")
    metadata = PackedWeightMetadata(
        logical_shape=(n, k),
        storage_layout=storage_layout or spec.storage_layout,
        pack_version=pack_version or spec.pack_version,
        weight_dtype=spec.weight_dtype,
        padded_k=padded,
        group_size=spec.group_size,
        packed_bits=packed_bits,
        nibble_order=nibble_order,
        nibble_signed=spec.symmetric,
        local_shape=local_shape,
        shard_axis=shard_axis,
    )
    return PackedWeight(
        qweight=qweight.contiguous(), scales=scales, zero_points=zero_points, metadata=metadata
    )


def validate_w4a16_packed_weight(
    weight: PackedWeight, *, spec: QuantSpec, logical_shape: tuple[int, int] | None = None
) -> None:
    """Strict ABI check before a W4A16 backend runs (layout.py:786-867).

    Raises ``TypeError`` / ``ValueError`` for the same conditions as xqt's
    validator: wrong layout tag, shape, group size outside {32,64,128}, nibble
    order, signedness vs ``spec.symmetric``, missing or surplus zero points.
    """

    if not hasattr(weight, "metadata") or not hasattr(weight, "qweight"):
        raise TypeError("W4A16 validation requires a PackedWeight")
    if spec.weight_dtype != "int4":
        raise ValueError("W4A16 validation requires QuantSpec.weight_dtype='int4'")
    meta = weight.metadata
    if meta.weight_dtype != "int4" or meta.packed_bits != 4:
        raise ValueError("W4A16 PackedWeight must contain packed 4-bit storage")
    if meta.storage_layout != W4_LAYOUT:
        raise ValueError(
            f"W4A16 backend requires storage_layout={W4_LAYOUT!r}, got {meta.storage_layout!r}"
        )
    if logical_shape is None:
        raise ValueError("W4A16 validation requires logical_shape=(N,K)")
    expected = (int(logical_shape[0]), int(logical_shape[1]))
    if tuple(meta.logical_shape) != expected:
        raise ValueError(
            f"W4A16 logical shape mismatch: metadata={meta.logical_shape}, expected={expected}"
        )
    n, k = expected
    if meta.padded_k < k:
        raise ValueError("W4A16 padded_k cannot be smaller than logical K")
    if meta.group_size not in {32, 64, 128}:
        raise ValueError("W4A16 canonical storage requires group_size 32, 64, or 128")
    if spec.group_size != meta.group_size:
        raise ValueError(
            f"W4A16 group_size mismatch: spec={spec.group_size}, metadata={meta.group_size}"
        )
    if meta.nibble_order != "low_high":
        raise ValueError("W4A16 canonical storage requires low_high nibble order")
    if meta.nibble_signed != spec.symmetric:
        raise ValueError(
            "W4A16 signedness mismatch: "
            f"metadata.nibble_signed={meta.nibble_signed}, spec.symmetric={spec.symmetric}"
        )
    if spec.symmetric and spec.weight_zero_point:
        raise ValueError("symmetric W4A16 cannot declare a weight zero point")
    if not spec.symmetric and not spec.weight_zero_point:
        raise ValueError("asymmetric W4A16 requires weight_zero_point=True")
    if not isinstance(weight.qweight, torch.Tensor):
        raise TypeError("W4A16 qweight must be a torch.Tensor")
    columns = (int(meta.padded_k) + 1) // 2
    if weight.qweight.dtype != torch.uint8 or tuple(weight.qweight.shape) != (n, columns):
        raise ValueError(
            f"W4A16 qweight must be uint8 with shape {(n, columns)}, got "
            f"dtype={weight.qweight.dtype}, shape={tuple(weight.qweight.shape)}"
        )
    _check_scale(weight.scales, shape=(n, int(meta.padded_k)), spec=spec, name="W4A16 scales")
    if spec.weight_zero_point:
        _check_scale(
            weight.zero_points, shape=(n, int(meta.padded_k)), spec=spec, name="W4A16 zero_points"
        )
    elif weight.zero_points is not None:
        raise ValueError("symmetric W4A16 must not carry zero_points")


# --------------------------------------------------------------------------------------
# HF AutoAWQ / AutoGPTQ int32 words -> canonical storage (layout.py:217-531)
# --------------------------------------------------------------------------------------


def unpack_int32_nibbles(words: torch.Tensor, *, awq_order: bool) -> torch.Tensor:
    """``[R,C]`` int32 words -> ``[R,C,8]`` codes in logical order."""

    if words.ndim != 2 or words.dtype not in _INT_DTYPES:
        raise TypeError("int32 packed weights must be a rank-2 integer tensor")
    shifts = torch.arange(0, 32, 4, device=words.device, dtype=torch.int64)
    codes = ((words.to(torch.int64).unsqueeze(-1) >> shifts) & 0x0F).to(torch.uint8)
    if awq_order:
        codes = codes[..., torch.tensor(AWQ_NIBBLE_ORDER, device=words.device)]
    return codes


def _source_codes(qweight: torch.Tensor, *, n: int, k: int, awq: bool) -> torch.Tensor:
    if qweight.ndim != 2:
        raise ValueError("source INT4 qweight must be rank-2")
    if qweight.dtype == torch.uint8 and qweight.shape[0] == n:
        return unpack_int4(qweight, logical_k=k, signed=False)
    if qweight.dtype not in {torch.int16, torch.int32, torch.int64}:
        raise TypeError("GPTQ/AWQ source qweight must be an int32-like tensor")
    codes = unpack_int32_nibbles(qweight, awq_order=awq)
    k_major = tuple(qweight.shape) == (k, (n + 7) // 8)      # AWQ native: [K, N/8]
    n_major = tuple(qweight.shape) == ((k + 7) // 8, n)      # GPTQ native: [K/8, N]
    # Each method prefers its native orientation when a square shape is ambiguous.
    if (awq and k_major) or (not awq and not n_major and k_major):
        return codes.reshape(k, -1)[:, :n].transpose(0, 1).contiguous()
    if n_major:
        return codes.permute(1, 0, 2).reshape(n, -1)[:, :k].contiguous()
    raise ValueError(
        f"unsupported INT4 qweight shape {tuple(qweight.shape)} for logical [N,K]=[{n},{k}]"
    )


def _group_parameter(value: torch.Tensor, *, n: int, groups: int, name: str) -> torch.Tensor:
    tensor = value.detach().to(torch.float32)
    if tensor.ndim == 3 and tensor.shape[-1] == 1:
        tensor = tensor[..., 0]
    if tensor.ndim == 1:
        if tensor.numel() == n:
            return tensor.reshape(n, 1).expand(n, groups).contiguous()
        if tensor.numel() == groups:
            return tensor.reshape(1, groups).expand(n, groups).contiguous()
    elif tensor.ndim == 2:
        if tuple(tensor.shape) == (n, groups):
            return tensor.contiguous()
        if tuple(tensor.shape) == (groups, n):
            return tensor.transpose(0, 1).contiguous()
        if tuple(tensor.shape) in {(n, 1), (1, groups)}:
            return tensor.expand(n, groups).contiguous()
    raise ValueError(f"{name} shape {tuple(value.shape)} is not [N,G] or [G,N]")


def _check_g_idx(g_idx: torch.Tensor | None, *, k: int, group_size: int) -> None:
    if g_idx is None:
        return
    expected = torch.arange(k, device=g_idx.device) // int(group_size)
    if g_idx.numel() != k or not torch.equal(g_idx.reshape(-1).to(expected.dtype), expected):
        raise ValueError("act-order (non-sequential g_idx) checkpoints are not supported")


def _group_zero_points(value, *, n: int, groups: int, awq: bool):
    if value is None:
        return None
    if value.dtype in {torch.int16, torch.int32, torch.int64} and tuple(value.shape) == (groups, (n + 7) // 8):
        # HF checkpoints pack qzeros like qweight: int32 words of eight nibbles along N.
        codes = unpack_int32_nibbles(value, awq_order=awq)
        return codes.reshape(groups, -1)[:, :n].transpose(0, 1).to(torch.float32).contiguous()
    return _group_parameter(value, n=n, groups=groups, name="zero_points")


def _canonical_w4(codes, *, n, k, scales, zero_points, group_size, signed, pack_version) -> PackedWeight:
    group = int(group_size)
    if group not in {32, 64, 128}:
        raise ValueError("W4A16 canonical repack supports group_size 32, 64, or 128")
    if tuple(codes.shape) != (n, k):
        raise ValueError(f"decoded INT4 codes must have shape {(n, k)}, got {tuple(codes.shape)}")
    padded_k = -(-k // group) * group
    groups = padded_k // group
    if padded_k != k:
        codes = torch.nn.functional.pad(codes, (0, padded_k - k), value=0)
    zeros = _group_zero_points(zero_points, n=n, groups=groups, awq=not signed)
    if signed:
        # GPTQ words hold offset-binary codes; canonical signed storage is value = code - 8
        # (padding columns therefore decode to -8, exactly as in layout.py:362-383).
        packed = pack_int4_signed(codes.to(torch.int16) - 8)
    else:
        packed = pack_int4_unsigned(codes)
    spec = QuantSpec(
        weight_dtype="int4",
        activation_dtype="fp16",
        output_dtype="fp16",
        weight_granularity="groupwise",
        group_size=group,
        symmetric=signed,
        weight_zero_point=zeros is not None,
        weight_scale_source="weight_offline",
    )
    return build_packed_weight(
        packed,
        logical_shape=(n, k),
        spec=spec,
        scales=_group_parameter(scales, n=n, groups=groups, name="scales"),
        zero_points=zeros,
        padded_k=padded_k,
        storage_layout=W4_LAYOUT,
        pack_version=pack_version,
    )


def repack_gptq_int4(
    qweight, *, logical_shape, scales, zero_points=None, group_size=128, g_idx=None,
    pack_version="xqt-w4a16-gptq-v1",
) -> PackedWeight:
    """GPTQ int32 words -> signed canonical W4 (layout.py:476-503)."""

    n, k = int(logical_shape[0]), int(logical_shape[1])
    if zero_points is not None:
        raise ValueError("GPTQ signed canonical INT4 does not support zero_points")
    _check_g_idx(g_idx, k=k, group_size=group_size)
    codes = _source_codes(qweight, n=n, k=k, awq=False)
    return _canonical_w4(codes, n=n, k=k, scales=scales, zero_points=None, group_size=group_size,
                         signed=True, pack_version=pack_version)


def repack_awq_int4(
    qweight, *, logical_shape, scales, zero_points=None, group_size=128, g_idx=None,
    pack_version="xqt-w4a16-awq-v1",
) -> PackedWeight:
    """AWQ int32 words -> unsigned canonical W4 with zero points (layout.py:506-531)."""

    n, k = int(logical_shape[0]), int(logical_shape[1])
    _check_g_idx(g_idx, k=k, group_size=group_size)
    codes = _source_codes(qweight, n=n, k=k, awq=True)
    return _canonical_w4(codes, n=n, k=k, scales=scales, zero_points=zero_points,
                         group_size=group_size, signed=False, pack_version=pack_version)


def signed_storage_to_unsigned(packed_signed: torch.Tensor) -> torch.Tensor:
    """Two's-complement nibbles -> offset codes with zero point 8.

    ``value = code - 8`` holds after flipping bit 3 of every nibble, i.e.
    ``byte ^ 0x88`` (xqt/runtime/modules/awq_w4a16_linear.py:25-71).
    """

    if packed_signed.dtype != torch.uint8:
        raise TypeError("signed INT4 storage must be uint8")
    return packed_signed ^ 0x88


__all__ = [
    "AWQ_NIBBLE_ORDER",
    "W4_LAYOUT",
    "W8_LAYOUT",
    "build_packed_weight",
    "expected_weight_scale_shape",
    "pack_int4_signed",
    "pack_int4_unsigned",
    "repack_awq_int4",
    "repack_gptq_int4",
    "signed_storage_to_unsigned",
    "unpack_int32_nibbles",
    "unpack_int4",
    "unpack_int4_signed",
    "validate_w4a16_packed_weight",
]
