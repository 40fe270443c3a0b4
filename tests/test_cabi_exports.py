"""The C-ABI library loads on a machine without a GPU and exports every declared symbol."""

from __future__ import annotations

import pathlib
import re

import pytest

from xqt_b200 import native

HEADER = pathlib.Path(__file__).resolve().parent.parent / "include" / "xqt_b200.h"


def declared_symbols() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(xqt_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_is_built_and_loads():
    assert native.LIBRARY_PATH.exists(), "run `python -m xqt_b200.build`"
    assert native.version().startswith("xqt-b200")


def test_every_declared_symbol_is_exported_and_bound():
    lib = native.library()
    names = declared_symbols()
    assert names, "no declarations parsed from the header"
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/xqt_b200.h but not exported"
        assert name in native.SIGNATURES, f"{name} has no ctypes prototype in xqt_b200.native"
    for name in native.SIGNATURES:
        assert name in names, f"{name} bound in python but not declared in the header"


def test_argument_checks_need_no_gpu():
    lib = native.library()
    assert lib.xqt_b200_w4a16_workspace_bytes(16, 4096, 4096) > 0
    assert lib.xqt_b200_w4a16_select_variant(16, 4096, 4096, 4096, 128, 0, 0) == native.VARIANT["gemv"]
    assert lib.xqt_b200_w4a16_select_variant(16, 4096, 4096, 4096, 64, 0, 0) == native.VARIANT["simt"]
    # invalid group size is rejected before any CUDA call
    code = lib.xqt_b200_w4a16_run(0, 0, 0, 0, 0, 0, 0, 4, 8, 64, 64, 48, 0, 1, 1, 1, 0, 0, 0, 0, 0)
    assert code == 1
    with pytest.raises(native.CudaCallError):
        native.check(code, "xqt_b200_w4a16_run")
    # M == 0 is a successful no-op
    assert lib.xqt_b200_w4a16_run(0, 0, 0, 0, 0, 0, 0, 0, 8, 64, 64, 64, 0, 1, 1, 1, 0, 0, 0, 0, 0) == 0
