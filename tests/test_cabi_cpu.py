"""CPU: the C-ABI library builds, loads and exports every symbol include/fba.h declares; host-side
argument validation answers with status codes (no GPU needed: those calls return before any launch)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    from flex_block_attn_b200 import _cabi
    from flex_block_attn_b200.build import build_library

    build_library()
    return _cabi.lib()


def declared_symbols():
    text = (ROOT / "include" / "fba.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fba_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib):
    from flex_block_attn_b200 import _cabi

    names = declared_symbols()
    assert "fba_fwd" in names and "fba_bwd" in names and "fba_build_index" in names
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/fba.h but not exported"
    assert set(_cabi.EXPORTED_SYMBOLS) <= set(names)


def test_abi_version(lib):
    assert lib.fba_abi_version() == 1


def test_bad_arguments_return_status_codes(lib):
    assert lib.fba_build_index(None, 2, 1, 1, 4, 4, None, None, None, None, None) == -1
    assert b"mask is null" in lib.fba_last_error()
    n1, n2 = ctypes.c_uint64(), ctypes.c_uint64()
    assert lib.fba_bwd_scratch_bytes(1, 2, 300, ctypes.byref(n1), ctypes.byref(n2)) == 0
    assert n1.value == 2 * 384 * 2 * 4 and n2.value == 2 * 384 * 128 * 4
    assert lib.fba_bwd_scratch_bytes(0, 2, 300, ctypes.byref(n1), ctypes.byref(n2)) == -1
    assert lib.fba_fwd(None, None, None, None, None, 1, 1, 1, 128, 128, None, None, None) == -1
    assert lib.fba_set_timing_events(3, None, None) == -1
    assert lib.fba_set_timing_events(0, None, None) == 0
    # entry points added beside the reference's interface: argument checks come before any CUDA call
    assert lib.fba_fwd_scaled(None, None, None, None, None, 1, 1, 1, 128, 128, None, 0.1, None, None) == -1
    assert lib.fba_bwd_scaled(*([None] * 9), 1, 1, 1, 128, 128, None, 0.1, None, None, None, None) == -1
    p = ctypes.c_void_p()
    assert lib.fba_peer_alloc(0, ctypes.byref(p)) == -1 and p.value is None
    assert lib.fba_peer_export(None, None) == -1 and lib.fba_peer_open(None, ctypes.byref(p)) == -1
    assert lib.fba_peer_free(None) == 0 and lib.fba_peer_close(None) == 0
    assert lib.fba_peer_exchange(None, None, 2, 0, 1, 2, 1, 1, 8, 1, 1, 1, 1, None) == -1
    assert b"fba_peer_exchange" in lib.fba_last_error()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from flex_block_attn_b200 import _cabi

    monkeypatch.setattr(_cabi, "_LIB", None)
    monkeypatch.setattr(_cabi, "LIB_PATH", tmp_path / "nope.so")
    monkeypatch.delenv("FBA_AUTO_BUILD", raising=False)
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _cabi.lib()
