"""The C-ABI library loads without a GPU and exports what include/dionw_b200.h declares."""

from __future__ import annotations

import ctypes
import re

from conftest import ROOT

from dionw_b200 import _native

HEADER = (ROOT / "include" / "dionw_b200.h").read_text()


def _declared() -> set[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    return set(re.findall(r"\b(dionw_[a-z0-9_]+)\s*\(", text))


def test_library_exports_every_declared_symbol() -> None:
    lib = ctypes.CDLL(str(_native.LIBRARY_PATH))
    declared = _declared()
    assert len(declared) >= 24
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_python_binding_covers_the_header() -> None:
    assert set(_native.SIGNATURES) == _declared()
    _native.library()  # sets argtypes for every entry: fails on a missing symbol


def test_version_and_error_text_work_without_a_gpu() -> None:
    lib = _native.library()
    assert b"sm_100a" in lib.dionw_version()
    assert _native.newton_schulz_workspace_bytes(2, 256, 1024, _native.NS_GRAM) > 2 * 256 * 1024 * 2
    assert _native.newton_schulz_workspace_bytes(0, 256, 1024, _native.NS_GRAM) == 0
    status = lib.dionw_select_rows(None, None, 0, 0, 0, None, None, None, None)
    assert status == -1
    assert "select_rows" in _native.last_error()
