"""ctypes binding of the C-ABI shared library (``include/xqt_b200.h``).

The library is built in-tree by :mod:`xqt_b200.build` as ``xqt_b200/libxqt_b200.so``.
There is no fallback: if the library is missing or a symbol is absent the call
raises :class:`NativeLibraryError`; a non-zero return code raises
:class:`CudaCallError`.  Both derive from ``XQTBackendError`` so xqt's GEMM
dispatcher records them and walks on to its next candidate
(xqt/kernels/ops/gemm/dispatch.py:253-257), exactly as for its sm_89 artifacts
(xqt/kernels/ops/_impl/gemm_backends/sm89/w4a16_sm89.py:61-78).
"""

from __future__ import annotations

import ctypes
import pathlib
import threading

import torch

from .errors import CudaCallError, NativeLibraryError

LIBRARY_PATH = pathlib.Path(__file__).resolve().parent / "libxqt_b200.so"

FP16, BF16, FP32 = 0, 1, 2
ACT = {"none": 0, "relu": 1, "gelu": 2, "silu": 3}
VARIANT = {"auto": 0, "simt": 1, "gemv": 2, "tcgen05": 3, "tcgen05_fused": 4}
VARIANT_NAMES = {value: key for key, value in VARIANT.items()}
DTYPE_CODE = {torch.float16: FP16, torch.bfloat16: BF16, torch.float32: FP32}

_P, _I, _Z = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t

# symbol -> (restype, argtypes); must list every function include/xqt_b200.h declares
SIGNATURES: dict[str, tuple] = {
    "xqt_b200_version": (ctypes.c_char_p, []),
    "xqt_b200_error_string": (ctypes.c_char_p, [_I]),
    "xqt_b200_device_supported": (_I, [_I]),
    "xqt_b200_w4a16_workspace_bytes": (_Z, [_I, _I, _I]),
    "xqt_b200_w4a16_select_variant": (_I, [_I] * 7),
    "xqt_b200_w4a16_two_pass": (_I, [_I]),
    "xqt_b200_w4a16_fused_preferred": (_I, [_I] * 5),
    "xqt_b200_w4a16_run": (_I, [_P] * 7 + [_I] * 10 + [_P, _Z, _I, _P]),
    "xqt_b200_w4a16_decode_workspace_bytes": (_Z, []),
    "xqt_b200_w4a16_decode_supported": (_I, [_I] * 4),
    "xqt_b200_w4a16_decode_tiled": (_I, [_P] * 6 + [_I] * 8 + [_P, _Z, _P]),
    "xqt_b200_w4a16_decode_tc_workspace_bytes": (_Z, []),
    "xqt_b200_w4a16_decode_tc_supported": (_I, [_I] * 4),
    "xqt_b200_w4a16_decode_tc": (_I, [_P] * 6 + [_I] * 8 + [_P, _Z, _P]),
    "xqt_b200_w4a16_decode_lanes_supported": (_I, [_I] * 4),
    "xqt_b200_w4a16_decode_lanes_plan": (_I, [_I] * 4 + [ctypes.POINTER(_I), ctypes.POINTER(_I)]),
    "xqt_b200_w4a16_decode_lanes_set_plan": (_I, [_I, _I]),
    "xqt_b200_w4a16_decode_lanes": (_I, [_P] * 7 + [_I] * 9 + [_P, _P]),
    "xqt_b200_w4a16_decode_lanes_select": (_I, [_P] * 7 + [_I] * 9 + [_P, _Z, _P, _P]),
    "xqt_b200_w4a16_decode_tiled_static": (_I, [_P] * 6 + [_I] * 8 + [_P]),
    "xqt_b200_w4a16_decode_static_scratch_bytes": (_Z, []),
    "xqt_b200_w4a16_decode_static_max_n": (_I, []),
    "xqt_b200_rotate_quantize": (_I, [_P] * 5 + [_I] * 7 + [_P]),
    "xqt_b200_quantize_per_tensor": (_I, [_P] * 4 + [_I] * 3 + [ctypes.c_float, _P]),
    "xqt_b200_w8a8_gemm": (_I, [_P] * 6 + [_I] * 4 + [_P, _Z, _P]),
    "xqt_b200_lowrank_down": (_I, [_P] * 4 + [_I] * 3 + [_P]),
    "xqt_b200_lowrank_up": (_I, [_P] * 3 + [_I] * 4 + [_P, _Z, _P]),
    "xqt_b200_w8a8_gemm_addend": (_I, [_P] * 7 + [_I] * 4 + [_P, _Z, _P]),
    "xqt_b200_w4a4_aux_tile_bytes": (_Z, [_I]),
    "xqt_b200_w4a4_supported": (_I, [_I] * 3),
    "xqt_b200_w4a4_workspace_bytes": (_Z, [_I] * 3),
    "xqt_b200_w4a4_gemm": (_I, [_P] * 8 + [_I] * 5 + [_P, _Z, _P]),
    "xqt_b200_w4a4_expand_weight": (_I, [_P, _P, _I, _I, _P]),
    "xqt_b200_w4a4_dense_workspace_bytes": (_Z, [_I] * 3),
    "xqt_b200_w4a4_dense_preferred": (_I, [_I] * 3),
    "xqt_b200_w4a4_dense": (_I, [_P] * 8 + [_I] * 4 + [_P, _Z, _P]),
    "xqt_b200_lowrank_down_tc": (_I, [_P] * 3 + [_I] * 3 + [_P, _Z, _P]),
    "xqt_b200_peer_allreduce": (_I, [_P, _P, _I, _I, ctypes.c_uint, ctypes.c_longlong, _I, _P, _P, _I, ctypes.c_uint, _P, _P]),
    "xqt_b200_peer_allgather_counted": (_I, [_P, _P, _I, _I, _P, ctypes.c_longlong, ctypes.c_longlong, _P, ctypes.c_uint, _P, _P]),
    "xqt_b200_peer_allreduce_counted": (_I, [_P, _P, _I, _I, _P, ctypes.c_longlong, ctypes.c_longlong, _I, _P, _P, _I, ctypes.c_uint, _P, _P]),
    "xqt_b200_w4a16_decode_static_status": (_I, [ctypes.POINTER(ctypes.c_uint), _P]),
    "xqt_b200_swiglu": (_I, [_P, _P, _I, _I, _I, _P]),
    "xqt_b200_workspace_status": (_I, [_P, ctypes.POINTER(ctypes.c_uint), _P]),
}

_lock = threading.Lock()
_library: ctypes.CDLL | None = None


def library() -> ctypes.CDLL:
    """Load (once) and return the shared library with typed prototypes."""

    global _library
    if _library is not None:
        return _library
    with _lock:
        if _library is not None:
            return _library
        if not LIBRARY_PATH.exists():
            raise NativeLibraryError(
                f"{LIBRARY_PATH} is missing: build it with `python -m xqt_b200.build` (needs nvcc)"
            )
        try:
            handle = ctypes.CDLL(str(LIBRARY_PATH))
        except OSError as exc:
            raise NativeLibraryError(f"cannot load {LIBRARY_PATH}: {exc}") from exc
        for name, (restype, argtypes) in SIGNATURES.items():
            try:
                function = getattr(handle, name)
            except AttributeError as exc:
                raise NativeLibraryError(f"{LIBRARY_PATH} lacks symbol {name}; rebuild it") from exc
            function.restype = restype
            function.argtypes = argtypes
        _library = handle
        return handle


def available() -> bool:
    """True when the library loads.  Says nothing about a GPU being present."""

    try:
        library()
    except NativeLibraryError:
        return False
    return True


def version() -> str:
    return library().xqt_b200_version().decode()


def check(code: int, symbol: str) -> None:
    if code != 0:
        detail = library().xqt_b200_error_string(int(code))
        raise CudaCallError(symbol, code, detail.decode() if detail else "")


def ptr(tensor: torch.Tensor | None) -> int:
    return 0 if tensor is None else tensor.data_ptr()


def stream_handle(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


# One scratch buffer per (device, stream): launches on one stream are ordered, so they may share
# it; launches on different streams may overlap and must not.
_workspaces: dict[tuple[int, int, str], torch.Tensor] = {}


def workspace(device: torch.device, nbytes: int, tag: str = "run") -> torch.Tensor:
    """Zero-initialised scratch of at least ``nbytes`` for the current stream of ``device``.

    ``tag`` separates kernel families whose scratch layouts differ: the decode kernels keep tickets
    that must stay zero between launches where the GEMM keeps a converted copy of the activations,
    so they never share a buffer."""

    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (index, stream_handle(device), tag)
    buffer = _workspaces.get(key)
    if buffer is None or buffer.numel() < nbytes:
        size = max(int(nbytes), 1 << 20)
        buffer = torch.zeros(size, dtype=torch.uint8, device=torch.device("cuda", index))
        _workspaces[key] = buffer
    return buffer


_status_words: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device 32-bit word (zero until a kernel's bounded wait runs out) handed to the entry
    points that take a status pointer instead of a workspace."""

    index = device.index if device.index is not None else torch.cuda.current_device()
    word = _status_words.get(index)
    if word is None:
        word = torch.zeros(64, dtype=torch.int32, device=torch.device("cuda", index))
        _status_words[index] = word
    return word


def workspace_status(device: torch.device) -> int:
    """Worst status word of the current stream's scratch buffers and of the device's status word
    (0 = every bounded wait completed)."""

    index = device.index if device.index is not None else torch.cuda.current_device()
    worst = 0
    word = _status_words.get(index)
    if word is not None:
        worst = int(word[0].item()) & 0xFFFFFFFF
    for (dev_index, stream, _tag), buffer in list(_workspaces.items()):
        if dev_index != index or stream != stream_handle(device):
            continue
        value = ctypes.c_uint(0)
        check(library().xqt_b200_workspace_status(buffer.data_ptr(), ctypes.byref(value), stream_handle(device)),
              "xqt_b200_workspace_status")
        worst = max(worst, int(value.value))
    return worst


__all__ = [
    "ACT", "BF16", "DTYPE_CODE", "FP16", "FP32", "LIBRARY_PATH", "SIGNATURES", "VARIANT", "VARIANT_NAMES",
    "available", "check", "library", "ptr", "status_word", "stream_handle", "version", "workspace", "workspace_status",
]
