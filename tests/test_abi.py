"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import re
from pathlib import Path

from infer_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols(header="infer_b200.h"):
    text = (ROOT / "include" / header).read_text()
    return sorted(set(re.findall(r"INFER_API[^;(]*?\b(infer_\w+)\s*\(", text)))


def test_header_declares_the_path():
    names = declared_symbols()
    for must in ("infer_kv_pool_create", "infer_kv_append", "infer_paged_decode", "infer_paged_prefill",
                 "infer_flash_attn_prefill", "infer_strerror"):
        assert must in names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared_symbols() + declared_symbols("infer_b200_selftest.h"):
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"


def test_bindings_cover_every_declared_symbol():
    assert sorted(_lib.SIGNATURES) == declared_symbols()
    assert sorted(_lib.SELFTEST_SIGNATURES) == declared_symbols("infer_b200_selftest.h")


def test_product_modules_do_not_reach_the_selftest_entry_points():
    """Only infer_b200/selftest.py (used by the tests) names the diagnostic entry points."""
    for path in (ROOT / "infer_b200").glob("*.py"):
        if path.name in ("selftest.py", "_lib.py"):
            continue
        assert "infer_selftest_" not in path.read_text(), path
    assert "infer_selftest_" not in (ROOT / "bench.py").read_text()


def test_error_strings_and_argument_checks_need_no_gpu():
    lib = _lib.load()
    assert lib.infer_abi_version() == 1
    assert lib.infer_strerror(0) == b"ok"
    for code in range(-8, 0):
        assert lib.infer_strerror(code) not in (b"ok", b"unknown error code")
    assert lib.infer_strerror(-99) == b"unknown error code"
    # argument validation happens before any CUDA call
    handle = ctypes.c_void_p()
    assert lib.infer_kv_pool_create(ctypes.byref(handle), None, None, None, None, 4, 256, 8, 128, 0) == _lib.ERR_NULL
    buf = ctypes.create_string_buffer(64)
    p = ctypes.cast(buf, ctypes.c_void_p)
    assert lib.infer_kv_pool_create(ctypes.byref(handle), p, p, None, None, 4, 100, 8, 128, 0) == _lib.ERR_GEOMETRY
    assert lib.infer_kv_pool_create(ctypes.byref(handle), p, p, None, None, 4, 256, 8, 64, 0) == _lib.ERR_GEOMETRY
    assert lib.infer_kv_pool_create(ctypes.byref(handle), p, p, None, None, 4, 256, 8, 128, 7) == _lib.ERR_DTYPE
    assert lib.infer_kv_pool_create(ctypes.byref(handle), p, p, None, None, 4, 256, 8, 128, 1) == _lib.ERR_NULL
    assert lib.infer_kv_append(None, p, p, 1024, 1024, p, 1, None, 0, None) == _lib.ERR_NULL
    assert lib.infer_paged_decode(None, p, p, p, p, 4, 1, 8, 0.1, None, 0, None) == _lib.ERR_NULL
    assert lib.infer_flash_attn_prefill(p, p, p, p, 1, 3, 2, 64, None) == _lib.ERR_GEOMETRY
    assert lib.infer_kv_append_workspace_bytes(None) == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    try:
        _lib.load()
    except ImportError as e:
        assert "no CPU or PyTorch fallback" in str(e)
    else:
        raise AssertionError("loading a missing library must raise")
