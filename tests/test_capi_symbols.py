"""The shared library loads without a GPU and exports every symbol the header declares."""
import ctypes
import re
from pathlib import Path

from oasr_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]


def _declared():
    text = (ROOT / "include" / "oasr_b200.h").read_text()
    return sorted(set(re.findall(r"OASR_API[^;(]*?\b(oasr_b200_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    names = _declared()
    assert len(names) >= 25
    assert "oasr_b200_gemm" in names and "oasr_b200_fmha_varlen" in names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    missing = [n for n in _declared() if not hasattr(lib, n)]
    assert not missing, f"missing exports: {missing}"


def test_binding_table_matches_header():
    assert sorted(_lib.exported_names()) == _declared()


def test_version_and_error_plumbing():
    assert "sm_100a" in _lib.version()
    # validation happens before any CUDA call, so it works without a GPU
    lib = _lib.load()
    rc = lib.oasr_b200_glu(None, None, 1, 8, _lib.DT_BF16, None)
    assert rc == _lib.ERR_INVALID and "null pointer" in _lib.last_error()
    rc = lib.oasr_b200_gemm(ctypes.c_void_p(16), ctypes.c_void_p(16), ctypes.c_void_p(16), None, 4, 5002, 64,
                            _lib.ACT_NONE, _lib.DT_BF16, None)
    assert rc == _lib.ERR_ALIGN and "8-aligned" in _lib.last_error()
    rc = lib.oasr_b200_set_tunable(b"nope", 1)
    assert rc == _lib.ERR_INVALID
