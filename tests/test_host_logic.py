"""CPU-only checks of the host side: the C-ABI library loads and exports every symbol the header
declares (no compute calls), struct layouts match, and the Python mirror keeps the reference's
closed-engine behaviour."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    import ane
    from ane import _ffi

    header = open(os.path.join(ROOT, "include", "ane_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(ane_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 30
    for name in sorted(declared):
        assert hasattr(_ffi.lib, name), f"libane_b200.so does not export {name}"
        assert name in _ffi.SIGNATURES, f"{name} has no ctypes signature"
    assert _ffi.lib.ane_version() >= 100
    assert os.path.basename(ane.LIB_PATH) == "libane_b200.so"


def test_struct_sizes_are_stable():
    from ane import _ffi

    assert ctypes.sizeof(_ffi.Options) == 168
    assert ctypes.sizeof(_ffi.StepResult) == 112
    assert ctypes.sizeof(_ffi.State) == 56


def test_open_rejects_bad_struct_size_without_a_gpu():
    from ane import _ffi

    o = _ffi.Options()
    o.struct_size = 4
    h = ctypes.c_void_p()
    rc = _ffi.lib.ane_open(ctypes.byref(o), None, 0, None, ctypes.byref(h))
    assert rc == -1 and not h.value
    assert b"struct_size" in _ffi.lib.ane_last_error(None)


def test_closed_engine_calls_fail_cleanly():
    from ane import _ffi

    assert _ffi.lib.ane_step(None, None) == -1
    assert _ffi.lib.ane_get_lr(None) == 0.0
    assert _ffi.lib.ane_close(None) == 0
    assert _ffi.lib.ane_tensor_size(None, 0, 0) == -1


def test_oracle_is_not_linked_into_the_product():
    import subprocess

    import ane

    out = subprocess.run(["ldd", ane.LIB_PATH], capture_output=True, text=True).stdout
    assert "oracle" not in out
    syms = subprocess.run(["nm", "-D", ane.LIB_PATH], capture_output=True, text=True).stdout
    assert "orc_" not in syms
    for root, _, files in os.walk(os.path.join(ROOT, "autoresearch-go-ane_b200")):
        if "/build" in root or "/lib" in root:
            continue
        for f in files:
            if f.endswith((".cu", ".cuh", ".h", ".py", ".go")):
                text = open(os.path.join(root, f), errors="ignore").read()
                assert "oracle" not in text.lower() or f == "__init__.py", f"{f} mentions the oracle"
