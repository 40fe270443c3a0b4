"""W4A16 linear on canonical ``xqt_int4_nk_v1`` tensors: the torch-facing call into the C ABI.

``w4a16_linear`` is registered as ``torch.ops.xqt_operator_opt.b200_w4a16_linear`` (xqt reserves
that namespace for its custom CUDA operators, xqt/kernels/wrappers/cuda_extension.py:20-85) with a
fake implementation for tracing; the real one only checks arguments, allocates the output and
hands raw pointers to ``xqt_b200_w4a16_run``.
"""

from __future__ import annotations

import torch

from .. import native
from ..errors import XQTBackendError
from ..weakid import WeakIdDict


def _check_cuda(name: str, tensor: torch.Tensor | None, device: torch.device) -> None:
    if tensor is None:
        return
    if not tensor.is_cuda or tensor.device != device:
        raise XQTBackendError(f"B200 W4A16 {name} must be a CUDA tensor on {device}")
    if not tensor.is_contiguous():
        raise XQTBackendError(f"B200 W4A16 {name} must be contiguous")


_integral_cache = WeakIdDict()      # zero-point tensor -> (version, answer); dies with the tensor


def _integer_zero_points(zero_points: torch.Tensor | None) -> bool:
    """True when every zero point is an integer in [0, 1000] (cached per tensor: one device sync
    the first time a weight is seen).  The tensor-core GEMM folds the zero point into an exact
    integer subtraction and is only valid then."""

    if zero_points is None:
        return True
    hit = _integral_cache.get(zero_points)
    if hit is None or hit[0] != zero_points._version:
        z = zero_points.to(torch.float32)
        hit = (zero_points._version, bool(((z == z.round()) & (z >= 0) & (z <= 1000)).all().item()))
        _integral_cache[zero_points] = hit
    return hit[1]


def select_variant(m: int, n: int, k: int, padded_k: int, group_size: int, activation: str = "none",
                   has_residual: bool = False) -> str:
    code = native.library().xqt_b200_w4a16_select_variant(
        m, n, k, padded_k, group_size, native.ACT[activation], int(has_residual))
    return native.VARIANT_NAMES[code]


def w4a16_linear(
    x: torch.Tensor,
    qweight: torch.Tensor,
    scales: torch.Tensor,
    zero_points: torch.Tensor | None = None,
    bias: torch.Tensor | None = None,
    residual: torch.Tensor | None = None,
    *,
    group_size: int,
    nibble_signed: bool,
    k: int | None = None,
    activation: str = "none",
    variant: str = "auto",
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
) -> torch.Tensor:
    """``y = x @ dequant(qweight).T (+bias) (+residual)`` with fp32 accumulation.

    ``out_dtype=torch.float32`` returns the unrounded sums (what a K-sharded layer reduces across
    ranks); it needs M > 16-style shapes the tensor-core GEMM covers and no residual.

    x ``[M,K]`` fp16/bf16; qweight ``uint8 [N, padded_K/2]``; scales / zero_points ``[N, G]``
    fp16/bf16/fp32 (same dtype); bias ``[N]`` (converted to fp32); residual ``[M,N]`` of x's dtype.
    """

    if x.ndim != 2 or x.dtype not in (torch.float16, torch.bfloat16):
        raise XQTBackendError("B200 W4A16 activation must be rank-2 fp16/bf16")
    device = x.device
    m, kx = int(x.shape[0]), int(x.shape[1])
    k = kx if k is None else int(k)
    if kx != k:
        raise XQTBackendError("B200 W4A16 activation K disagrees with the weight's logical K")
    if qweight.ndim != 2 or qweight.dtype != torch.uint8:
        raise XQTBackendError("B200 W4A16 qweight must be uint8 [N, padded_K/2]")
    n, padded_k = int(qweight.shape[0]), int(qweight.shape[1]) * 2
    groups = padded_k // int(group_size)
    if scales.dtype not in native.DTYPE_CODE or tuple(scales.shape) != (n, groups):
        raise XQTBackendError(f"B200 W4A16 scales must be [{n},{groups}] fp16/bf16/fp32")
    if zero_points is not None and (zero_points.dtype != scales.dtype or zero_points.shape != scales.shape):
        raise XQTBackendError("B200 W4A16 zero_points must match scales in shape and dtype")
    if activation not in native.ACT:
        raise XQTBackendError(f"B200 W4A16 unknown epilogue activation {activation!r}")
    if bias is not None:
        if bias.numel() != n:
            raise XQTBackendError("B200 W4A16 bias must have N elements")
        bias = bias.reshape(-1).to(device=device, dtype=torch.float32).contiguous()
    if residual is not None and (residual.dtype != x.dtype or tuple(residual.shape) != (m, n)):
        raise XQTBackendError("B200 W4A16 residual must be [M,N] in the activation dtype")
    for name, tensor in (("activation", x), ("qweight", qweight), ("scales", scales),
                         ("zero_points", zero_points), ("residual", residual)):
        _check_cuda(name, tensor, device)
    odt = x.dtype if out_dtype is None else out_dtype
    if odt not in (x.dtype, torch.float32):
        raise XQTBackendError("B200 W4A16 out_dtype must be the activation dtype or float32")
    if out is None:
        out = torch.empty((m, n), device=device, dtype=odt)
    elif out.dtype != odt or tuple(out.shape) != (m, n) or not out.is_contiguous() or out.device != device:
        raise XQTBackendError("B200 W4A16 out must be a contiguous [M,N] tensor of the output dtype")
    if m == 0:
        return out
    lib = native.library()
    two_pass = bool(lib.xqt_b200_w4a16_two_pass(m))   # large M: fp32 dequantisation pass, any zero point
    if odt == torch.float32:
        if not two_pass and not _integer_zero_points(zero_points):
            raise XQTBackendError("fp32 partial sums need the tensor-core GEMM, i.e. integer zero points")
        # unrounded partial sums of a K-sharded layer: the fused form where it is preferred (it writes fp32 as well), else two-pass
        fused_ok = variant in ("auto", "tcgen05_fused") and activation == "none" and residual is None \
            and _integer_zero_points(zero_points) and lib.xqt_b200_w4a16_fused_preferred(m, n, k, padded_k, int(group_size))
        variant = "tcgen05_fused" if fused_ok else "tcgen05"
    if variant == "auto":
        variant = select_variant(m, n, k, padded_k, int(group_size), activation, residual is not None)
        if variant == "tcgen05" and not two_pass and not _integer_zero_points(zero_points):
            variant = "simt"
        # the fused single-pass form where it measures faster (17 <= M <= 512); integer zero points only
        if variant == "tcgen05" and odt != torch.float32 and lib.xqt_b200_w4a16_fused_preferred(m, n, k, padded_k, int(group_size)) \
                and _integer_zero_points(zero_points):
            variant = "tcgen05_fused"
    if variant == "tcgen05_fused" and not _integer_zero_points(zero_points):
        raise XQTBackendError("the single-pass tcgen05 GEMM needs integer zero points")
    scratch = native.workspace(device, lib.xqt_b200_w4a16_workspace_bytes(m, n, k))
    stream = native.stream_handle(device)
    act_code, param_code = native.DTYPE_CODE[x.dtype], native.DTYPE_CODE[scales.dtype]

    with torch.cuda.device(device):
        code = lib.xqt_b200_w4a16_run(
            x.data_ptr(), qweight.data_ptr(), scales.data_ptr(), native.ptr(zero_points), native.ptr(bias),
            native.ptr(residual), out.data_ptr(), m, n, k, padded_k, int(group_size), int(bool(nibble_signed)),
            act_code, param_code, native.DTYPE_CODE[odt], native.ACT[activation], scratch.data_ptr(), scratch.numel(),
            native.VARIANT[variant], stream)
    native.check(code, "xqt_b200_w4a16_run")
    return out


def bind_w4a16_linear(
    qweight: torch.Tensor,
    scales: torch.Tensor,
    zero_points: torch.Tensor | None = None,
    *,
    rows: int,
    dtype: torch.dtype,
    group_size: int,
    nibble_signed: bool,
    k: int | None = None,
    bias: torch.Tensor | None = None,
    variant: str = "auto",
):
    """Validate the static tensors once and return ``run(x, out=None) -> Tensor`` for a fixed
    row count, the way ``bind_awq_w4a16_decode`` does for the sm_89 decode kernel
    (xqt/kernels/ops/_impl/cuda/awq_w4a16_sm89.py:217-302): the closure only checks the
    activation and makes one C-ABI call.  The scratch buffer is the one of the stream that is
    current when the closure runs for the first time."""

    device = qweight.device
    probe = torch.empty((rows, int(qweight.shape[1]) * 2 if k is None else int(k)), device=device, dtype=dtype)
    w4a16_linear(probe[:0], qweight, scales, zero_points, bias, None, group_size=group_size,
                 nibble_signed=nibble_signed, k=k, variant=variant)          # argument validation only
    n, padded_k = int(qweight.shape[0]), int(qweight.shape[1]) * 2
    kk = padded_k if k is None else int(k)
    lib = native.library()
    fn = lib.xqt_b200_w4a16_run
    bias32 = None if bias is None else bias.reshape(-1).to(device=device, dtype=torch.float32).contiguous()
    nbytes = lib.xqt_b200_w4a16_workspace_bytes(rows, n, kk)
    static = (qweight.data_ptr(), scales.data_ptr(), native.ptr(zero_points), native.ptr(bias32), 0)
    tail = (rows, n, kk, padded_k, int(group_size), int(bool(nibble_signed)), native.DTYPE_CODE[dtype],
            native.DTYPE_CODE[scales.dtype], native.DTYPE_CODE[dtype], 0)
    variant_code = native.VARIANT[variant]
    index = device.index if device.index is not None else torch.cuda.current_device()
    keep = (qweight, scales, zero_points, bias32)

    def run(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        if x.dtype != dtype or x.ndim != 2 or x.shape[0] != rows or x.shape[1] != kk or not x.is_contiguous() \
                or x.device != device:
            raise XQTBackendError("bound B200 W4A16 call: activation shape, dtype, device or layout mismatch")
        if torch.cuda.current_device() != index:
            raise XQTBackendError("bound B200 W4A16 call: make the weight's device current before calling")
        if out is None:
            out = torch.empty((rows, n), device=device, dtype=dtype)
        scratch = native.workspace(device, nbytes)
        code = fn(x.data_ptr(), *static, out.data_ptr(), *tail, scratch.data_ptr(), scratch.numel(),
                  variant_code, torch.cuda.current_stream(device).cuda_stream)
        if code != 0:
            native.check(code, "xqt_b200_w4a16_run")
        return out

    run.keep = keep          # the callable owns the tensors whose raw pointers it passes
    return run


def decode_supported(m: int, n: int, k: int, group_size: int) -> bool:
    return bool(native.library().xqt_b200_w4a16_decode_supported(int(m), int(n), int(k), int(group_size)))


def glu_row_order(inter: int) -> torch.Tensor:
    """Row permutation of a horizontally fused ``[gate; up]`` weight (``2*inter`` rows) that puts, into every 128-row
    tile, 64 gate rows followed by their 64 up rows -- the order the decode kernel's fused SwiGLU epilogue expects."""

    if inter % 64:
        raise XQTBackendError("fused SwiGLU decode needs the intermediate size to be a multiple of 64")
    base = torch.arange(inter).reshape(inter // 64, 1, 64)
    return torch.cat((base, base + inter), dim=1).reshape(-1)


def bind_w4a16_decode(tiled, *, rows: int, dtype: torch.dtype, bias: torch.Tensor | None = None,
                      out_dtype: torch.dtype | None = None, glu: bool = False, out_select: tuple[int, int] | None = None):
    """Hot-callable for the decode kernel on a :class:`xqt_b200.prepack.TiledW4` layer:
    ``run(x, out=None, residual=None) -> Tensor`` for a fixed row count (1..16).  Static tensors are
    validated here, once; each call checks the activation and makes one C-ABI call
    (cf. ``bind_awq_w4a16_decode``, xqt/kernels/ops/_impl/cuda/awq_w4a16_sm89.py:217-302).

    ``glu`` (``lanes`` layout): the layer is a fused gate/up projection whose rows were laid out with
    :func:`glu_row_order`; the kernel's epilogue gates them, ``run`` returns ``silu(gate) * up`` as ``[rows, N/2]``
    with the bits of the unfused linear -> SwiGLU (the horizontally fused gate/up + SwiGLU of
    xqt/kernels/ops/_impl/cute/convrot_w8a8_sm89.py:664-917, at decode sizes).

    ``out_select = (device word address, stride in bytes)`` (``lanes`` layout): the kernel writes at
    ``out + ((word + 1) & 1) * stride`` -- the slot of a two-slot buffer that the counted peer reduction reads next
    (:class:`xqt_b200.parallel.PeerAllReduce`, ``counted=True``)."""

    device = tiled.weights.device
    if device.type != "cuda":
        raise XQTBackendError("B200 W4A16 decode needs the tiled layer on a CUDA device")
    if dtype not in (torch.float16, torch.bfloat16):
        raise XQTBackendError("B200 W4A16 decode supports fp16 or bf16 activations")
    n, k = tiled.n, tiled.k
    odt = dtype if out_dtype is None else out_dtype
    if odt not in (dtype, torch.float32):
        raise XQTBackendError("B200 W4A16 decode out_dtype must be the activation dtype or float32")
    lib = native.library()
    use_tc = tiled.layout == "rows128"
    if tiled.layout == "lanes":
        return _bind_decode_lanes(tiled, rows=rows, dtype=dtype, bias=bias, odt=odt, glu=glu, out_select=out_select)
    if glu or out_select is not None:
        raise XQTBackendError("the fused SwiGLU epilogue and the device-selected output slot are served by the lanes decode layout only")
    if use_tc:
        if not tiled.integer_zero_points:
            raise XQTBackendError("the tcgen05 decode kernel needs integer zero points in [0, 119]")
        supported = bool(lib.xqt_b200_w4a16_decode_tc_supported(rows, n, k, tiled.group_size))
    else:
        supported = decode_supported(rows, n, k, tiled.group_size)
    if not supported:
        raise XQTBackendError(f"B200 W4A16 decode does not cover M={rows}, N={n}, K={k}, group={tiled.group_size}")
    if tiled.params.dtype not in native.DTYPE_CODE or not tiled.weights.is_contiguous() or not tiled.params.is_contiguous():
        raise XQTBackendError("B200 W4A16 decode: tiled tensors must be contiguous, params fp16/bf16/fp32")
    bias32 = None if bias is None else bias.reshape(-1).to(device=device, dtype=torch.float32).contiguous()
    if bias32 is not None and bias32.numel() != n:
        raise XQTBackendError("B200 W4A16 bias must have N elements")
    head = (tiled.weights.data_ptr(), tiled.params.data_ptr(), native.ptr(bias32))
    if use_tc:
        fn, symbol = lib.xqt_b200_w4a16_decode_tc, "xqt_b200_w4a16_decode_tc"
        nbytes = lib.xqt_b200_w4a16_decode_tc_workspace_bytes()
        tail = (rows, n, k, tiled.group_size, int(tiled.nibble_signed), native.DTYPE_CODE[dtype],
                native.DTYPE_CODE[tiled.params.dtype], native.DTYPE_CODE[odt])
    else:
        if odt != dtype:
            raise XQTBackendError("fp32 output needs the tcgen05 decode layout (rows128)")
        fn, symbol = lib.xqt_b200_w4a16_decode_tiled, "xqt_b200_w4a16_decode_tiled"
        nbytes = lib.xqt_b200_w4a16_decode_workspace_bytes()
        tail = (rows, n, k, tiled.group_size, int(tiled.nibble_signed), int(tiled.has_zero_point),
                native.DTYPE_CODE[dtype], native.DTYPE_CODE[tiled.params.dtype])
    index = device.index if device.index is not None else torch.cuda.current_device()
    keep = (tiled, bias32)

    def run(x: torch.Tensor, out: torch.Tensor | None = None, residual: torch.Tensor | None = None) -> torch.Tensor:
        if x.dtype != dtype or x.ndim != 2 or x.shape[0] != rows or x.shape[1] != k or not x.is_contiguous() \
                or x.device != device:
            raise XQTBackendError("bound B200 W4A16 decode: activation shape, dtype, device or layout mismatch")
        if torch.cuda.current_device() != index:
            raise XQTBackendError("bound B200 W4A16 decode: make the weight's device current before calling")
        if out is None:
            out = torch.empty((rows, n), device=device, dtype=odt)
        if residual is not None and (residual.dtype != dtype or tuple(residual.shape) != (rows, n)
                                     or not residual.is_contiguous()):
            raise XQTBackendError("bound B200 W4A16 decode: residual must be contiguous [M,N] in the activation dtype")
        scratch = native.workspace(device, nbytes, "decode")
        code = fn(x.data_ptr(), *head, native.ptr(residual), out.data_ptr(), *tail, scratch.data_ptr(),
                  scratch.numel(), torch.cuda.current_stream(device).cuda_stream)
        if code != 0:
            native.check(code, symbol)
        return out

    run.keep = keep          # the callable owns the tensors whose raw pointers it passes
    return run


def _bind_decode_lanes(tiled, *, rows: int, dtype: torch.dtype, bias: torch.Tensor | None, odt: torch.dtype, glu: bool = False,
                       out_select: tuple[int, int] | None = None):
    """``bind_w4a16_decode`` for the ``lanes`` layout (cluster split-K kernel: no workspace)."""

    device = tiled.weights.device
    n, k = tiled.n, tiled.k
    if glu and (n % 128 or odt != dtype):
        raise XQTBackendError("fused SwiGLU decode: N must be a multiple of 128 and the output in the activation dtype")
    n_out = n // 2 if glu else n
    lib = native.library()
    if not lib.xqt_b200_w4a16_decode_lanes_supported(rows, n, k, tiled.group_size):
        raise XQTBackendError(f"B200 W4A16 decode does not cover M={rows}, N={n}, K={k}, group={tiled.group_size}")
    if tiled.params.dtype not in native.DTYPE_CODE or not tiled.weights.is_contiguous() or not tiled.params.is_contiguous():
        raise XQTBackendError("B200 W4A16 decode: tiled tensors must be contiguous, params fp16/bf16/fp32")
    bias32 = None if bias is None else bias.reshape(-1).to(device=device, dtype=torch.float32).contiguous()
    if bias32 is not None and bias32.numel() != n:
        raise XQTBackendError("B200 W4A16 bias must have N elements")
    if out_select is not None and glu:
        raise XQTBackendError("the device-selected output slot does not combine with the fused SwiGLU epilogue")
    fn = lib.xqt_b200_w4a16_decode_lanes if out_select is None else lib.xqt_b200_w4a16_decode_lanes_select
    head = (tiled.weights.data_ptr(), tiled.params[0].data_ptr(),
            tiled.params[1].data_ptr() if tiled.has_zero_point else 0, native.ptr(bias32))
    tail = (rows, n, k, tiled.group_size, int(tiled.nibble_signed), native.DTYPE_CODE[dtype],
            native.DTYPE_CODE[tiled.params.dtype], native.DTYPE_CODE[odt], 2 if glu else 0)
    if out_select is not None:
        tail = tail + (int(out_select[0]), int(out_select[1]))
    index = device.index if device.index is not None else torch.cuda.current_device()
    status = native.status_word(device)
    status_ptr = status.data_ptr()
    keep = (tiled, bias32, status)

    def run(x: torch.Tensor, out: torch.Tensor | None = None, residual: torch.Tensor | None = None) -> torch.Tensor:
        if x.dtype != dtype or x.ndim != 2 or x.shape[0] != rows or x.shape[1] != k or not x.is_contiguous() \
                or x.device != device:
            raise XQTBackendError("bound B200 W4A16 decode: activation shape, dtype, device or layout mismatch")
        if torch.cuda.current_device() != index:
            raise XQTBackendError("bound B200 W4A16 decode: make the weight's device current before calling")
        if out is None:
            out = torch.empty((rows, n_out), device=device, dtype=odt)
        elif tuple(out.shape) != (rows, n_out) or out.dtype != odt or not out.is_contiguous():
            raise XQTBackendError("bound B200 W4A16 decode: out must be contiguous [M, N] (N/2 with glu) in the output dtype")
        if residual is not None and (glu or residual.dtype != dtype or tuple(residual.shape) != (rows, n)
                                     or not residual.is_contiguous() or odt != dtype):
            raise XQTBackendError("bound B200 W4A16 decode: residual must be contiguous [M,N] in the activation dtype (none with glu)")
        code = fn(x.data_ptr(), *head, native.ptr(residual), out.data_ptr(), *tail, status_ptr,
                  torch.cuda.current_stream(device).cuda_stream)
        if code != 0:
            native.check(code, "xqt_b200_w4a16_decode_lanes")
        return out

    run.keep = keep          # the callable owns the tensors whose raw pointers it passes
    return run


def prepare_decode(qweight: torch.Tensor, scales: torch.Tensor, zero_points: torch.Tensor | None, *,
                   group_size: int, nibble_signed: bool, k: int | None = None, layout: str = "auto"):
    """Build the decode execution layout of a canonical W4 layer.  ``auto``: the cluster split-K
    layout (``lanes``) when the layer qualifies (group 64/128, K a multiple of 128 within the
    kernel's range); else the tcgen05 layout (``rows128``: group 64/128, integer zero points); else
    the stream-K mma.sync layout (``tile128``).  A layout name forces that layout."""

    from .. import prepack

    n, kk = int(qweight.shape[0]), int(qweight.shape[1]) * 2 if k is None else int(k)
    if layout not in ("auto", "lanes", "rows128", "tile128"):
        raise XQTBackendError(f"unknown decode layout {layout!r}")
    if layout == "lanes" or (layout == "auto" and group_size in (64, 128) and kk % 128 == 0 and
                             native.library().xqt_b200_w4a16_decode_lanes_supported(16, n, kk, int(group_size))):
        return prepack.lanes_w4(qweight, scales, zero_points, group_size=group_size, nibble_signed=nibble_signed, k=k)
    if layout == "tile128":
        return prepack.tile_w4(qweight, scales, zero_points, group_size=group_size, nibble_signed=nibble_signed, k=k)
    if layout == "rows128":
        return prepack.rows_w4(qweight, scales, zero_points, group_size=group_size, nibble_signed=nibble_signed, k=k)
    if group_size in (64, 128):
        tiled = prepack.rows_w4(qweight, scales, zero_points, group_size=group_size, nibble_signed=nibble_signed, k=k)
        if tiled.integer_zero_points:
            return tiled
    return prepack.tile_w4(qweight, scales, zero_points, group_size=group_size, nibble_signed=nibble_signed, k=k)


def w4a16_decode_tiled(x: torch.Tensor, tiled, bias=None, residual=None, out=None) -> torch.Tensor:
    """One-shot form of :func:`bind_w4a16_decode`."""

    return bind_w4a16_decode(tiled, rows=int(x.shape[0]), dtype=x.dtype, bias=bias)(x, out, residual)


def _register() -> None:
    """Expose the op under xqt's reserved custom-op namespace; harmless if already present."""

    try:
        op = torch.library.custom_op(
            "xqt_operator_opt::b200_w4a16_linear", mutates_args=(), device_types="cuda"
        )(_custom_op_entry)
        op.register_fake(_custom_op_fake)
    except Exception:  # noqa: BLE001 - re-import in one process, or torch without custom_op
        pass


def _custom_op_entry(x: torch.Tensor, qweight: torch.Tensor, scales: torch.Tensor,
                     zero_points: torch.Tensor | None, bias: torch.Tensor | None,
                     residual: torch.Tensor | None, group_size: int, nibble_signed: bool,
                     activation: str) -> torch.Tensor:
    return w4a16_linear(x, qweight, scales, zero_points, bias, residual, group_size=group_size,
                        nibble_signed=nibble_signed, activation=activation)


def _custom_op_fake(x, qweight, scales, zero_points, bias, residual, group_size, nibble_signed, activation):
    return x.new_empty((x.shape[0], qweight.shape[0]))


_register()

__all__ = ["bind_w4a16_decode", "bind_w4a16_linear", "decode_supported", "glu_row_order", "prepare_decode", "select_variant",
           "w4a16_decode_tiled",
           "w4a16_linear"]
