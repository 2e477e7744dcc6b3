"""The C-ABI library builds, loads, and exports every symbol include/lh_b200.h declares
(no compute calls: this runs without a GPU)."""

import os
import re
import subprocess

from conftest import ROOT

from lighthouse_b200 import _native


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "lh_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lh_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_symbols() == sorted(_native.EXPORTED_SYMBOLS)


def test_library_exports_every_declared_symbol(native_lib):
    out = subprocess.run(["nm", "-D", "--defined-only", str(_native.lib_path())], capture_output=True, text=True, check=True).stdout
    exported = set(re.findall(r"\sT\s+(lh_b200_[a-z0-9_]+)", out))
    missing = [s for s in declared_symbols() if s not in exported]
    assert not missing, f"declared in lh_b200.h but not exported: {missing}"
    for name in declared_symbols():
        assert hasattr(native_lib, name)


def test_struct_layouts_match_the_header():
    """ctypes mirrors of lh_memref_t / lh_view_t / lh_op_t have the sizes the C side computes."""
    import ctypes

    assert ctypes.sizeof(_native.MemRef) == 8 + 8 + 8 + 4 + 4 + 8 * 4 + 8 * 4
    assert ctypes.sizeof(_native.View) == 4 * 4 + 8 + 8 * 4 + 8 * 4
    assert ctypes.sizeof(_native.Op) == 4 * 4 + 4 * 2 + ctypes.sizeof(_native.View) * 8
    assert ctypes.sizeof(_native.ArgSig) == 8


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    import pytest

    monkeypatch.setenv("LH_B200_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_native, "_lib", None)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _native.load()


def test_errors_without_a_device_are_reported_not_swallowed(native_lib):
    """ctx creation on a machine without a GPU (or with a bad ordinal) returns an error code
    and a message; nothing falls back to the host."""
    import ctypes

    h = ctypes.c_void_p()
    rc = native_lib.lh_b200_ctx_create(10_000, ctypes.byref(h))
    assert rc != 0 and not h.value
    assert native_lib.lh_b200_last_error(None)
