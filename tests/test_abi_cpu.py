"""CPU checks of the boundary: the library loads, exports every symbol
include/svodb.h declares, and the header and the ctypes table agree. No
compute call is made (there is no GPU here)."""
import ctypes
import re
from pathlib import Path

import pytest

from svod_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "svodb.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(svodb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_what_the_binding_types():
    assert declared_symbols() == sorted(name for name, _, _ in _lib.SYMBOLS)


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_version_and_status_strings_without_a_device():
    lib = _lib.load()
    assert lib.svodb_version().startswith(b"svodb")
    assert lib.svodb_last_error() is not None
    assert lib.svodb_attention_workspace_bytes(2, 5, 4, 64, 3) == 4 * 3 * 2 * 5 * 4 * (64 + 2)
    assert lib.svodb_attention_workspace_bytes(2, 5, 4, 64, 1) == 0
    # split-K: [tiles][2] counters rounded up to 256 bytes, then [tiles][splits][2][128][256] f32
    assert lib.svodb_linear_workspace_bytes(512, 4096, 2) == 256 + 32 * 2 * 2 * 128 * 256 * 4
    assert lib.svodb_linear_workspace_bytes(700, 1000, 3) == 256 + 12 * 3 * 2 * 128 * 256 * 4
    assert lib.svodb_linear_workspace_bytes(512, 4096, 1) == 0


def test_struct_layouts_match_the_header():
    # svodb_tensor: pointer, two i32, 5 + 5 i64
    assert ctypes.sizeof(_lib.Tensor) == 8 + 4 + 4 + 80
    assert _lib.LinearOpts.into_at.offset % 8 == 0
    assert _lib.AttnOpts.workspace_bytes.offset % 8 == 0


def test_no_product_module_imports_the_oracle():
    for path in (ROOT / "svod_b200").rglob("*.py"):
        assert "oracle" not in path.read_text(), path


def test_the_error_latch_without_a_device():
    """A sticky CUDA error code (faked: no device is touched) makes every later
    call fail fast with SVODB_ERR_POISONED until the self-test clears it."""
    lib = _lib.load()
    assert lib.svodb_selftest_latch_error(0) == _lib.OK
    assert lib.svodb_selftest_latch_error(1) == _lib.ERR_LAUNCH            # cudaErrorInvalidValue: not sticky
    assert lib.svodb_selftest_latch_error(0) == _lib.OK
    assert lib.svodb_selftest_latch_error(700) == _lib.ERR_LAUNCH          # cudaErrorIllegalAddress: sticky
    try:
        assert lib.svodb_selftest_latch_error(0) == _lib.ERR_POISONED
        assert lib.svodb_graph_begin(None) == _lib.ERR_POISONED
        assert b"poisoned" in lib.svodb_last_error()
    finally:
        lib.svodb_selftest_clear_latch()
    assert lib.svodb_selftest_latch_error(0) == _lib.OK
