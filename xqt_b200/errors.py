"""Error types raised by the B200 backend.

The names follow xqt's leaf error module (xqt/core/base/errors.py:4-29): the GEMM
dispatcher catches ``XQTBackendError`` from an executor, records the reason and
moves on to the next registry candidate (xqt/kernels/ops/gemm/dispatch.py:253-257).
When xqt itself is importable the classes below are aliases of xqt's own, so an
error raised here is caught by xqt's dispatcher unchanged.
"""

from __future__ import annotations

try:  # pragma: no cover - only when the host project is installed next to us
    from xqt.core.base.errors import XQTBackendError, XQTError  # type: ignore
except Exception:  # noqa: BLE001 - absent or partially importable host project

    class XQTError(Exception):
        """Base error of the operator path."""

    class XQTBackendError(XQTError):
        """A native backend is missing or rejected the request."""


class NativeLibraryError(XQTBackendError):
    """The C-ABI shared library is absent, stale or lacks a symbol."""


class CudaCallError(XQTBackendError):
    """A C-ABI entry point returned a non-zero CUDA error code."""

    def __init__(self, symbol: str, code: int, detail: str = "") -> None:
        self.symbol = symbol
        self.code = int(code)
        message = f"{symbol} failed with CUDA error {code}"
        if detail:
            message = f"{message}: {detail}"
        super().__init__(message)


__all__ = ["CudaCallError", "NativeLibraryError", "XQTBackendError", "XQTError"]
