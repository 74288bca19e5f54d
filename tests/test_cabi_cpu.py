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
    assert lib.fba_abi_version() == 2


def test_bad_arguments_return_status_codes(lib):
    assert lib.fba_build_index(None, 2, 1, 1, 4, 4, None, None, None, None, None) == -1
    assert b"mask is null" in lib.fba_last_error()
    n1, n2 = ctypes.c_uint64(), ctypes.c_uint64()
    assert lib.fba_bwd_scratch_bytes(1, 2, 300, ctypes.byref(n1), ctypes.byref(n2)) == 0
    assert n1.value == 2 * 384 * 2 * 4 and n2.value == 2 * 384 * 128 * 4
    assert lib.fba_bwd_scratch_bytes(0, 2, 300, ctypes.byref(n1), ctypes.byref(n2)) == -1
    assert lib.fba_fwd(None, None, None, None, None, 1, 1, 1, 128, 128, None, None, None) == -1
    assert lib.fba_set_timing_events(4, None, None) == -1
    assert lib.fba_set_timing_events(0, None, None) == 0
    # entry points added beside the reference's interface: argument checks come before any CUDA call
    assert lib.fba_fwd_scaled(None, None, None, None, None, 1, 1, 1, 128, 128, None, 0.1, None, None) == -1
    assert lib.fba_bwd_scaled(*([None] * 9), 1, 1, 1, 128, 128, None, 0.1, None, None, None, None) == -1
    # the reference-shaped entry points, the work order, the status helpers
    n = ctypes.c_uint64()
    assert lib.fba_attn_workspace_bytes(1, 2, 2, 1536, 1536, 384, 384, 2, 0, ctypes.byref(n)) == 0
    assert n.value == 256 * 3                              # 4x4 idx, 4 cnt, 6 order entries: one 256-byte slot each
    assert lib.fba_attn_workspace_bytes(1, 2, 2, 1536, 1536, 384, 384, 2, 1, ctypes.byref(n)) == 0
    assert n.value == 256 * 3 + 2 * 1536 * 2 * 4 + 2 * 1536 * 128 * 4
    assert lib.fba_attn_workspace_bytes(1, 2, 2, 1536, 1536, 384, 384, 3, 0, ctypes.byref(n)) == -1
    assert b"block_mask dim must be 2/4" in lib.fba_last_error()
    assert lib.fba_attn_workspace_bytes(1, 2, 2, 1536, 1536, 100, 384, 2, 0, ctypes.byref(n)) == -1
    assert lib.fba_attn_workspace_bytes(1, 2, 2, 1500, 1536, 384, 384, 2, 0, ctypes.byref(n)) == -1
    assert lib.fba_attn_forward(*([None] * 5), 1, 1, 1, 128, 128, 128, 128, None, None, 2, 0, None, 0, None, None) == -1
    assert lib.fba_attn_backward(*([None] * 9), 1, 1, 1, 128, 128, 128, 128, None, None, 2, 0, None, 0, None, None) == -1
    assert lib.fba_fwd_order(None, 1, 1, 128, None, None) == -1
    assert lib.fba_bwd_order(None, 1, 2, 1, 128, None, None) == -1
    assert lib.fba_bwd_order(None, 1, 3, 2, 128, None, None) == -1
    assert lib.fba_check_status(None, None) == -1
    assert lib.fba_selftest_wait_timeout(None, 1000, None, None) == -1
    p = ctypes.c_void_p()
    assert lib.fba_peer_alloc(0, ctypes.byref(p)) == -1 and p.value is None
    assert lib.fba_peer_export(None, None) == -1 and lib.fba_peer_open(None, ctypes.byref(p)) == -1
    assert lib.fba_peer_free(None) == 0 and lib.fba_peer_close(None) == 0
    assert lib.fba_peer_exchange(None, None, 2, 0, 1, 2, 1, 1, 8, 1, 1, 1, 1, None) == -1
    assert b"fba_peer_exchange" in lib.fba_last_error()


def test_list_geometry_is_checked_before_any_device_work(lib):
    """A list whose entries / rows stand for groups of tiles must cover whole groups: a sequence that
    ends inside a group would make the kernels touch tiles (and backward scratch) past its end.
    The pointers below are never dereferenced: the checks answer first."""
    from flex_block_attn_b200._cabi import FbaList

    fake = ctypes.c_void_p(0x1000)
    def lst(stride, rows, rows_div, sub):
        return FbaList(0x1000, 0x1000, None, stride, rows, rows, rows_div, sub)
    # forward: Skv = 640 -> 5 key tiles, entries of 3 tiles (kv_block 384) do not divide it
    l = lst(2, 2, 1, 3)
    assert lib.fba_fwd(fake, fake, fake, fake, fake, 1, 1, 1, 256, 640, ctypes.byref(l), fake, None) == -1
    assert b"multiple of q2k->sub" in lib.fba_last_error()
    # forward: Sq = 640 -> 5 query tiles, list rows of 3 tiles do not divide it
    l = lst(2, 2, 3, 1)
    assert lib.fba_fwd(fake, fake, fake, fake, fake, 1, 1, 1, 640, 256, ctypes.byref(l), fake, None) == -1
    # a list that does not cover the sequence at all
    l = lst(1, 1, 1, 1)
    assert lib.fba_fwd(fake, fake, fake, fake, fake, 1, 1, 1, 256, 256, ctypes.byref(l), fake, None) == -1
    assert b"does not cover" in lib.fba_last_error()
    # backward: the mirrored pair for the key-major list
    l = lst(2, 2, 1, 3)
    args = [fake] * 9 + [1, 1, 1, 640, 256, ctypes.byref(l), fake, fake, fake, None]
    assert lib.fba_bwd(*args) == -1 and b"multiple of k2q->sub" in lib.fba_last_error()
    l = lst(2, 2, 3, 1)
    args = [fake] * 9 + [1, 1, 1, 256, 640, ctypes.byref(l), fake, fake, fake, None]
    assert lib.fba_bwd(*args) == -1
    # sizes the kernels do not support, and the dQ mode
    l = lst(1, 1, 1, 1)
    assert lib.fba_fwd(fake, fake, fake, fake, fake, 1, 1, 1, 64, 64, ctypes.byref(l), fake, None) == -1
    assert b"below 128" in lib.fba_last_error()
    assert lib.fba_fwd(fake, fake, fake, fake, fake, 1024, 64, 64, 128, 128, ctypes.byref(l), fake, None) == -5
    args = [fake] * 9 + [1, 1, 1, 128, 128, ctypes.byref(l), None, ctypes.c_float(0.1), 7, fake, fake, fake, None]
    assert lib.fba_bwd_ex(*args) == -1 and b"dq_mode" in lib.fba_last_error()
    args[17] = 1   # FBA_DQ_QMAJOR without a q2k list
    assert lib.fba_bwd_ex(*args) == -1 and b"q2k" in lib.fba_last_error()
    assert lib.fba_set_bwd_kernel(0) == -1
    # the work order refuses more items per (batch, head) than its shared-memory sort holds; callers then
    # leave `order` NULL (the Python layer does)
    big = FbaList(0x1000, 0x1000, None, 16, 13000, 13000, 1, 1)
    assert lib.fba_bwd_order(ctypes.byref(big), 1, 1, 1, 13000 * 128, fake, None) == -5
    assert b"12288" in lib.fba_last_error()
    assert lib.fba_fwd_order(ctypes.byref(big), 1, 1, 2 * 12288 * 128, fake, None) == -1   # list does not cover Sq


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from flex_block_attn_b200 import _cabi

    monkeypatch.setattr(_cabi, "_LIB", None)
    monkeypatch.setattr(_cabi, "LIB_PATH", tmp_path / "nope.so")
    monkeypatch.delenv("FBA_AUTO_BUILD", raising=False)
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _cabi.lib()


def test_setup_py_builds_the_library_into_the_package(tmp_path, lib):
    """`setup.py build_py` (what `pip install .` runs) compiles for sm_100a and ships the .so."""
    import subprocess
    import sys

    out = tmp_path / "lib"
    r = subprocess.run([sys.executable, "setup.py", "-q", "build_py", "--build-lib", str(out)], cwd=ROOT,
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    pkg = out / "flex_block_attn_b200"
    assert (pkg / "libfba_b200.so").exists() and (pkg / "interface.py").exists() and (pkg / "csrc" / "fba_fwd.cu").exists()
    from flex_block_attn_b200.build import NVCC_FLAGS

    archs = [f for f in NVCC_FLAGS if "arch=" in f or f.startswith("-arch")]
    assert archs == ["arch=compute_100a,code=sm_100a"]
